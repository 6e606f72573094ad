"""Rollout decode throughput of the engine (continuous batching over the paged KV cache) with
synthetic prompts and random-init weights:

    python -m prime_rl_b200.engine.bench_decode --model qwen3-30b-a3b --batch 256 --prompt 1024 --steps 32

Prefills ``batch`` prompts of ``prompt`` uniform-random token ids, then times ``steps`` engine
steps in which every sequence decodes one token (temperature 1.0 sampling, logprobs returned),
through the same ``Engine.step`` the HTTP server drives. Prints one JSON line with decode
tokens/s (wall clock around the timed steps, which end with the device-to-host read of the
sampled tokens) and the prefill rate.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch

from ..models import build_model, resolve_arch
from .engine import Engine, Request
from .sampler import SamplingParams


def run_decode(model: str = "qwen3-30b-a3b", batch: int = 256, prompt: int = 1024, steps: int = 32, warmup: int = 4,
               layers: int | None = None, fp8: bool = False, graphs: bool = True, dev: torch.device | None = None,
               tp=None) -> dict | None:
    """Builds the engine, prefills ``batch`` prompts and times ``steps`` decode steps. ``tp``: an
    ``engine/tp.py`` context for a tensor-parallel engine (ranks other than 0 follow and return None)."""
    arch = resolve_arch(model)
    if layers:
        arch = arch.model_copy(update={"num_hidden_layers": layers})
    if dev is None:
        dev = tp.device if tp is not None else torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    world = tp.size if tp is not None else 1
    net = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0)
    # requests admitted early keep decoding while the rest is prefilled: give every request enough
    # budget to still be running in the timed region
    prefill_steps = (batch * prompt + 16383) // 16384 + 1
    budget = prefill_steps + warmup + steps + 4
    total = prompt + budget + 2
    pages = batch * ((total + 15) // 16 + 1) + 64
    eng = Engine(net, num_pages=pages, page_size=16, max_running=batch, max_prefill_tokens=16384,
                 enable_prefix_cache=False, use_cuda_graphs=graphs, max_model_len=total + 16,
                 weight_dtype="fp8" if fp8 else "bf16", tp=tp)
    if tp is not None and tp.rank != 0:
        eng.follow()
        return None
    g = torch.Generator().manual_seed(0)
    params = SamplingParams(temperature=1.0, max_tokens=budget)
    for _ in range(batch):
        eng.submit(Request(prompt=torch.randint(0, arch.vocab_size, (prompt,), generator=g).tolist(), params=params))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while eng.waiting or eng._inbox:
        eng.step()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    n0 = eng.stats["generation_tokens"]
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    toks = eng.stats["generation_tokens"] - n0
    from ..ops import _runtime as rt

    rt.check_status()
    if tp is not None:
        eng.shutdown()
    return {"metric": "rollout decode tokens/s", "model": model, "layers": arch.num_hidden_layers,
            "batch": batch, "mean_running": toks / steps, "prompt_len": prompt, "steps": steps,
            "decode_tokens_per_s": toks / dt, "ms_per_step": 1e3 * dt / steps,
            "prefill_tokens_per_s": batch * prompt / t_prefill,
            "peak_memory_gib": torch.cuda.max_memory_allocated() / 2**30, "n_gpus": world,
            "parallelism": f"tp{world}" if world > 1 else "single",
            "dtype": "fp8 weights / bf16 KV" if fp8 else "bf16", "cuda_graphs": graphs,
            "data": "synthetic (uniform random token ids, random-init weights)"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--layers", type=int, default=None, help="debug: truncate the model")
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 weights (128x128 scales), 1x128 activation scales")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step kernel by kernel")
    args = ap.parse_args(argv)
    # under torchrun with N processes: one tensor-parallel engine over N GPUs (rank 0 drives and reports)
    tp = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from .tp import init_tp

        tp = init_tp(16384 + args.prompt, resolve_arch(args.model).hidden_size)
    res = run_decode(args.model, args.batch, args.prompt, args.steps, args.warmup, args.layers, args.fp8,
                     not args.no_graphs, tp=tp)
    if res is not None:
        print(json.dumps(res), flush=True)
    if tp is not None:
        tp.close()


if __name__ == "__main__":
    main()
