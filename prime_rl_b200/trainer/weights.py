"""HuggingFace safetensors import / export.

Export writes ``model-0000i-of-0000n.safetensors`` shards of at most ``max_shard_bytes`` plus
``model.safetensors.index.json`` and ``config.json``; whole decoder layers stay in one shard
(reference: src/prime_rl/utils/weights.py:45-252). LoRA runs export a PEFT adapter directory
(``adapter_model.safetensors`` + ``adapter_config.json``) instead.
"""

from __future__ import annotations

import json
import re
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..models import convert


def _layer_key(name: str) -> str:
    m = re.match(r"(model\.layers\.\d+)\.", name)
    return m.group(1) if m else name.split(".")[0]


def plan_shards(sizes: dict[str, int], max_shard_bytes: int) -> list[list[str]]:
    """Greedy packing of tensors into shards that keeps each decoder layer together."""
    groups: dict[str, list[str]] = {}
    for n in sizes:
        groups.setdefault(_layer_key(n), []).append(n)
    shards: list[list[str]] = [[]]
    cur = 0
    for _, names in groups.items():
        g = sum(sizes[n] for n in names)
        if shards[-1] and cur + g > max_shard_bytes:
            shards.append([])
            cur = 0
        shards[-1].extend(names)
        cur += g
    return [s for s in shards if s]


def _is_expert_hf_key(name: str) -> bool:
    return re.search(r"\.experts\.\d+\.", name) is not None


@torch.no_grad()
def save_hf_checkpoint(model, out_dir: Path, *, max_shard_bytes: int = 5 * 2 ** 30, dtype=torch.bfloat16,
                       tokenizer_dir: Path | None = None) -> Path:
    """Replicated model: call on one rank. Expert-parallel model: a collective, every rank calls it;
    the ranks of the exporting ep group each write the experts they own (numbered globally) into files
    of their own, the first of them also writes everything else and the merged index."""
    out_dir = Path(out_dir)
    info = convert.expert_parallel_info(model)
    if info is not None:
        return _save_hf_expert_parallel(model, out_dir, info, max_shard_bytes, dtype, tokenizer_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    sd = convert.model_state(model, "hf")
    index = _write_shards(sd, out_dir, "model", max_shard_bytes, dtype)
    (out_dir / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
    _write_config(model, out_dir, tokenizer_dir)
    return out_dir


def _write_shards(sd: dict, out_dir: Path, stem: str, max_shard_bytes: int, dtype) -> dict:
    sizes = {k: v.numel() * torch.empty((), dtype=dtype).element_size() for k, v in sd.items()}
    shards = plan_shards(sizes, max_shard_bytes)
    index = {"metadata": {"total_size": sum(sizes.values())}, "weight_map": {}}
    for i, names in enumerate(shards):
        fname = f"{stem}.safetensors" if len(shards) == 1 else f"{stem}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file({n: sd[n].detach().to("cpu", dtype).contiguous() for n in names}, str(out_dir / fname),
                  metadata={"format": "pt"})
        for n in names:
            index["weight_map"][n] = fname
    return index


def _save_hf_expert_parallel(model, out_dir: Path, info, max_shard_bytes, dtype, tokenizer_dir) -> Path:
    import torch.distributed as dist

    leader = info["writer"] and info["ep_rank"] == 0
    if leader:
        out_dir.mkdir(parents=True, exist_ok=True)
    dist.barrier()
    index = None
    if info["writer"]:
        sd = convert.model_state(model, "hf")               # this rank's experts under their global numbers
        mine = {k: v for k, v in sd.items() if _is_expert_hf_key(k) or leader}
        index = _write_shards(mine, out_dir, f"model-ep{info['ep_rank']:02d}", max_shard_bytes, dtype)
        parts = [None] * info["ep"]
        dist.all_gather_object(parts, index, group=info["group"])
        if leader:
            merged = {"metadata": {"total_size": sum(p["metadata"]["total_size"] for p in parts)}, "weight_map": {}}
            for p in parts:
                merged["weight_map"].update(p["weight_map"])
            (out_dir / "model.safetensors.index.json").write_text(json.dumps(merged, indent=2))
            _write_config(model, out_dir, tokenizer_dir)
    dist.barrier()
    return out_dir


def _write_config(model, out_dir: Path, tokenizer_dir: Path | None) -> None:
    (out_dir / "config.json").write_text(json.dumps(model.arch.to_hf_config(), indent=2))
    if tokenizer_dir is not None:
        import shutil

        for f in Path(tokenizer_dir).glob("token*"):
            shutil.copy(f, out_dir / f.name)


@torch.no_grad()
def save_lora_adapter(model, out_dir: Path, rank: int, alpha: float, target_modules: list[str]) -> Path:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    if convert.expert_parallel_info(model) is not None:
        raise NotImplementedError("LoRA adapter export of an expert-parallel model: gather the adapters first "
                                  "(convert.model_state(..., gather_experts=True)) or train the adapters with ep = 1")
    sd = {k: v.detach().to("cpu").contiguous() for k, v in convert.lora_to_peft(model).items()}
    save_file(sd, str(out_dir / "adapter_model.safetensors"), metadata={"format": "pt"})
    (out_dir / "adapter_config.json").write_text(json.dumps({
        "peft_type": "LORA", "r": rank, "lora_alpha": alpha, "target_modules": target_modules, "bias": "none",
        "task_type": "CAUSAL_LM", "lora_dropout": 0.0}, indent=2))
    return out_dir


def read_hf_state(path: Path, device: str = "cpu") -> dict[str, torch.Tensor]:
    path = Path(path)
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    out: dict[str, torch.Tensor] = {}
    for f in files:
        if f.name.startswith("adapter_"):
            continue
        with safe_open(str(f), framework="pt", device=device) as sf:
            for k in sf.keys():
                out[k] = sf.get_tensor(k)
    return out


@torch.no_grad()
def load_hf_checkpoint(model, path: Path, strict: bool = True) -> None:
    sd = read_hf_state(path)
    if model.arch.tie_word_embeddings:
        sd.pop("lm_head.weight", None)
    convert.load_model_state(model, sd, "hf", strict=strict)


_VISION_PREFIXES = ("model.visual.", "visual.", "model.vision_tower.", "vision_tower.")


@torch.no_grad()
def load_vision_tower(tower, path: Path, strict: bool = True) -> int:
    """Fills ``models/vision.py: VisionTower`` from the ``visual.*`` tensors of a HF checkpoint directory (the tower's
    parameter names are the checkpoint's). Returns the number of tensors loaded; 0 when the checkpoint has none
    (a text-only checkpoint: the tower keeps its initial values)."""
    path = Path(path)
    want = tower.state_dict()
    got: dict[str, torch.Tensor] = {}
    for f in sorted(path.glob("*.safetensors")):
        if f.name.startswith("adapter_"):
            continue
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for k in sf.keys():
                for pre in _VISION_PREFIXES:
                    if k.startswith(pre) and k[len(pre):] in want:
                        got[k[len(pre):]] = sf.get_tensor(k)
                        break
    if not got:
        return 0
    missing = [k for k in want if k not in got and not k.endswith("inv_freq")]
    if missing and strict:
        raise KeyError(f"vision tower tensors missing from {path}: {missing[:5]}{' ...' if len(missing) > 5 else ''}")
    for k, t in got.items():
        if tuple(t.shape) != tuple(want[k].shape):
            raise ValueError(f"vision tower tensor {k}: checkpoint {tuple(t.shape)} vs model {tuple(want[k].shape)}")
        want[k].copy_(t.to(want[k].dtype))
    return len(got)
