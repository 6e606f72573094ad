"""HF bf16 safetensors directory -> block-scaled fp8 (e4m3, 128 x 128 scales in
``<name>_scale_inv``) with the matching ``quantization_config`` in ``config.json``
(reference: src/prime_rl/tools/convert_bf16_to_fp8.py).

    python -m prime_rl_b200.tools.convert_bf16_to_fp8 <src_dir> <dst_dir> [--device cuda]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from ..models.fp8 import quantize_state_dict
from ._io import read_dir, write_dir

QUANT_CONFIG = {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic", "weight_block_size": [128, 128]}


def convert(src: Path, dst: Path, device: str = "cpu") -> Path:
    sd = {k: v.to(device) for k, v in read_dir(src).items()}
    out = quantize_state_dict(sd)
    cfg_path = Path(src) / "config.json"
    config = json.loads(cfg_path.read_text()) if cfg_path.exists() else {}
    config["quantization_config"] = QUANT_CONFIG
    return write_dir(out, dst, src_dir=src, config=config)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("src", type=Path)
    ap.add_argument("dst", type=Path)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    print(convert(a.src, a.dst, a.device))


if __name__ == "__main__":
    main()
