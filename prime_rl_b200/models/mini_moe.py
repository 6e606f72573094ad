"""Builds a small random-weight model of any supported family, writes it as a HuggingFace-style
checkpoint directory (``config.json`` + ``model.safetensors``) and checks that the
HF -> native -> HF conversion reproduces every tensor and that a reloaded model computes the
same hidden states. Useful as a download-free stand-in for a real checkpoint in pipelines and
as a conversion self-check when a family is added
(reference: scripts/mini_moe.py).

    python -m prime_rl_b200.models.mini_moe --arch tiny-glm-moe-dsa --output-dir /tmp/mini --verify
    python -m prime_rl_b200.models.mini_moe --arch qwen3-30b-a3b --layers 2 --hidden 256 --output-dir /tmp/mini
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import convert
from .config import ModelArch, resolve_arch
from .layers import SeqInfo
from .model import build_model


def shrink(arch: ModelArch, layers: int | None, hidden: int | None, experts: int | None, vocab: int | None) -> ModelArch:
    upd: dict = {}
    if layers is not None:
        upd["num_hidden_layers"] = layers
        for f in ("layer_types", "block_types", "mixer_types", "mlp_layer_types", "heads_per_layer"):
            v = getattr(arch, f)
            if v is not None:
                upd[f] = list(v[:layers])
        upd["index_share_layers"] = [i for i in arch.index_share_layers if i < layers]
    if hidden is not None:
        upd.update(hidden_size=hidden, intermediate_size=2 * hidden,
                   moe_intermediate_size=max(64, hidden // 2) if arch.is_moe else 0)
    if experts is not None and arch.is_moe:
        upd.update(num_experts=experts, num_experts_per_tok=min(arch.num_experts_per_tok, experts))
    if vocab is not None:
        upd["vocab_size"] = vocab
    return arch.model_copy(update=upd)


def write_checkpoint(model, out_dir: Path) -> dict[str, torch.Tensor]:
    from safetensors.torch import save_file

    out_dir.mkdir(parents=True, exist_ok=True)
    sd = {k: v.detach().contiguous().clone() for k, v in convert.model_state(model, "hf").items()}
    save_file(sd, str(out_dir / "model.safetensors"), metadata={"format": "pt"})
    (out_dir / "config.json").write_text(json.dumps(model.arch.to_hf_config(), indent=2))
    return sd


def verify(model, out_dir: Path) -> None:
    from safetensors.torch import load_file

    sd = load_file(str(out_dir / "model.safetensors"))
    arch = ModelArch.from_pretrained(out_dir)
    other = build_model(arch, device="cpu", dtype=next(model.parameters()).dtype, seed=12345)
    convert.load_model_state(other, sd, "hf")
    again = convert.model_state(other, "hf")
    bad = [k for k in sd if not torch.equal(sd[k], again[k])]
    if bad:
        raise SystemExit(f"conversion round trip changed {len(bad)} tensors, e.g. {bad[:3]}")
    ids = torch.arange(24) % arch.vocab_size
    seq = SeqInfo.from_lengths([10, 14], "cpu")
    with torch.no_grad():
        a, b = model(ids, seq), other(ids, SeqInfo.from_lengths([10, 14], "cpu"))
    if not torch.allclose(a.float(), b.float(), atol=1e-4, rtol=1e-3):
        raise SystemExit("the reloaded model computes different hidden states")


def verify_engine(model, tokens: int = 8) -> float:
    """The rollout engine on this model against the model's own forward: greedy samples of a few prompts must be the
    arg-max of the forward over the finished sequences; returns the largest log-probability difference."""
    from ..engine.engine import Engine
    from ..engine.sampler import SamplingParams

    arch = model.arch
    model.eval()
    eng = Engine(model, num_pages=256, page_size=16, max_model_len=256)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (19, 40, 6)]
    out = eng.generate_sync(prompts, SamplingParams(max_tokens=tokens, temperature=0.0))
    worst = 0.0
    dev = next(model.parameters()).device
    for p, r in zip(prompts, out):
        ids = torch.tensor(p + r.output, device=dev)
        with torch.no_grad():
            h = model(ids, SeqInfo.from_lengths([len(ids)], dev))
            lp = torch.log_softmax(h.float() @ model.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            t = len(p) - 1 + i
            if int(lp[t].argmax()) != tok and model.output_weight.dtype == torch.float32:
                raise SystemExit(f"the engine sampled token {tok} where the forward prefers {int(lp[t].argmax())}")
            worst = max(worst, abs(float(lp[t, tok]) - r.logprobs[i]))
    return worst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", required=True, help="a preset name or a local HF directory")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=None)
    ap.add_argument("--experts", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=None)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--verify-engine", action="store_true",
                    help="also run the rollout engine on the model and compare its samples with the model's forward")
    args = ap.parse_args(argv)
    arch = shrink(resolve_arch(args.arch), args.layers, args.hidden, args.experts, args.vocab)
    model = build_model(arch, device="cpu", dtype=getattr(torch, args.dtype), seed=args.seed)
    out = Path(args.output_dir)
    sd = write_checkpoint(model, out)
    n = sum(v.numel() for v in sd.values())
    print(f"{arch.model_type}: {len(sd)} tensors, {n / 1e6:.1f} M parameters -> {out}")
    if args.verify:
        verify(model, out)
        print("round trip verified")
    if args.verify_engine:
        print(f"rollout engine verified: largest log-probability difference {verify_engine(model):.2e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
