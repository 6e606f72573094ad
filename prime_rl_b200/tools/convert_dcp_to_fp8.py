"""Trainer checkpoint (DCP) -> HF block-scaled fp8 safetensors directory
(reference: src/prime_rl/tools/convert_dcp_to_fp8.py). Arguments as ``convert_dcp_to_bf16``."""

from __future__ import annotations

from .convert_dcp_to_bf16 import main as _main


def main(argv=None):
    _main(argv, fp8=True)


if __name__ == "__main__":
    main()
