"""Block-scaled fp8 safetensors directory -> bf16 (drops ``*_scale_inv`` and the
``quantization_config``; reference: src/prime_rl/tools/convert_fp8_to_bf16.py).

    python -m prime_rl_b200.tools.convert_fp8_to_bf16 <src_dir> <dst_dir>
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..models.fp8 import dequantize_state_dict
from ._io import read_dir, write_dir


def convert(src: Path, dst: Path) -> Path:
    out = dequantize_state_dict(read_dir(src), torch.bfloat16)
    cfg_path = Path(src) / "config.json"
    config = json.loads(cfg_path.read_text()) if cfg_path.exists() else {}
    config.pop("quantization_config", None)
    return write_dir(out, dst, src_dir=src, config=config)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("src", type=Path)
    ap.add_argument("dst", type=Path)
    a = ap.parse_args(argv)
    print(convert(a.src, a.dst))


if __name__ == "__main__":
    main()
