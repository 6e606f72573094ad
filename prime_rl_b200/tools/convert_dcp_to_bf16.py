"""Trainer checkpoint (DCP, prime-layout names under ``app.model``) -> HF bf16 safetensors
directory, without building the model or touching a GPU
(reference: src/prime_rl/tools/convert_dcp_to_bf16.py).

    python -m prime_rl_b200.tools.convert_dcp_to_bf16 <ckpt_dir>/step_N <dst_dir> --model qwen3-30b-a3b
    python -m prime_rl_b200.tools.convert_dcp_to_fp8  ...   (same arguments, fp8 output)
"""

from __future__ import annotations

import argparse
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp

from ..models import convert as conv
from ..models import resolve_arch
from ._io import write_dir


def read_dcp_model(step_dir: Path) -> dict[str, torch.Tensor]:
    """All tensors stored under ``app.model`` (full, unsharded values)."""
    reader = dcp.FileSystemReader(str(step_dir))
    meta = reader.read_metadata()
    sd = {}
    for key, m in meta.state_dict_metadata.items():
        if key.startswith("app.model.") and hasattr(m, "size"):
            sd[key] = torch.empty(m.size, dtype=m.properties.dtype)
    nested: dict = {"app": {"model": {k[len("app.model."):]: v for k, v in sd.items()}}}
    dcp.load(nested, checkpoint_id=str(step_dir), no_dist=True)
    return nested["app"]["model"]


def convert(step_dir: Path, dst: Path, model: str, fp8: bool = False) -> Path:
    arch = resolve_arch(model)
    prime = {k: v for k, v in read_dcp_model(Path(step_dir)).items() if "lora_" not in k}
    hf = {k: v.to(torch.bfloat16) for k, v in conv.prime_to_hf(prime, arch).items()}
    config = arch.to_hf_config()
    if fp8:
        from ..models.fp8 import quantize_state_dict
        from .convert_bf16_to_fp8 import QUANT_CONFIG

        hf = quantize_state_dict(hf)
        config["quantization_config"] = QUANT_CONFIG
    return write_dir(hf, dst, config=config)


def main(argv=None, fp8: bool = False):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("step_dir", type=Path)
    ap.add_argument("dst", type=Path)
    ap.add_argument("--model", required=True, help="preset name or path of a config.json")
    a = ap.parse_args(argv)
    print(convert(a.step_dir, a.dst, a.model, fp8=fp8))


if __name__ == "__main__":
    main()
