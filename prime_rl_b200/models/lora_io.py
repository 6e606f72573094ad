"""Loading PEFT-layout LoRA adapters into a model (the engine's ``/load_lora_adapter``)."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from .layers import LoRAAdapter
from .model import apply_lora


@torch.no_grad()
def load_peft_adapter(model, path: Path) -> None:
    path = Path(path)
    cfg = json.loads((path / "adapter_config.json").read_text())
    if not any(isinstance(m, LoRAAdapter) for m in model.modules()):
        apply_lora(model, cfg["r"], cfg["lora_alpha"], cfg["target_modules"])
    tensors = {}
    with safe_open(str(path / "adapter_model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    for name, mod in model.named_modules():
        if not isinstance(mod, LoRAAdapter):
            continue
        owner = name.rsplit(".", 1)[0]
        parent = owner.rsplit(".", 1)[0] if "." in owner else ""
        is_expert = name.endswith("lora_gate_up") or name.endswith("lora_down")
        r = mod.rank
        for s, member in enumerate(mod.names):
            target = f"{owner}.{member}" if is_expert else f"{parent}.{member}"
            a = tensors.get(f"base_model.model.{target}.lora_A.weight")
            b = tensors.get(f"base_model.model.{target}.lora_B.weight")
            if a is None or b is None:
                raise KeyError(f"adapter is missing weights for {target}")
            mod.lora_A[..., s * r:(s + 1) * r, :].copy_(a.to(mod.lora_A.dtype))
            mod.lora_B[s].copy_(b.to(mod.lora_B[s].dtype))
