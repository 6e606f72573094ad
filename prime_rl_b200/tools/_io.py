"""Shared helpers of the checkpoint conversion tools: sharded safetensors directories."""

from __future__ import annotations

import json
import shutil
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

from ..trainer.weights import plan_shards


def read_dir(path: Path) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    files = sorted(Path(path).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    for f in files:
        out.update(load_file(str(f)))
    return out


def write_dir(sd: dict[str, torch.Tensor], out_dir: Path, *, src_dir: Path | None = None, config: dict | None = None,
              max_shard_bytes: int = 5 * 2 ** 30) -> Path:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    sizes = {k: v.numel() * v.element_size() for k, v in sd.items()}
    shards = plan_shards(sizes, max_shard_bytes)
    index = {"metadata": {"total_size": sum(sizes.values())}, "weight_map": {}}
    for i, names in enumerate(shards):
        fname = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file({n: sd[n].detach().cpu().contiguous() for n in names}, str(out_dir / fname), metadata={"format": "pt"})
        for n in names:
            index["weight_map"][n] = fname
    (out_dir / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
    if config is not None:
        (out_dir / "config.json").write_text(json.dumps(config, indent=2))
    if src_dir is not None:
        for f in Path(src_dir).iterdir():
            if f.is_file() and f.suffix != ".safetensors" and f.name != "model.safetensors.index.json" and \
                    not (config is not None and f.name == "config.json"):
                shutil.copy(f, out_dir / f.name)
    return out_dir
