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
    arch = resolve_arch(args.model)
    if args.layers:
        arch = arch.model_copy(update={"num_hidden_layers": args.layers})
    # under torchrun with N processes: one tensor-parallel engine over N GPUs (rank 0 drives and reports)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    tp = None
    if world > 1:
        from .tp import init_tp

        tp = init_tp(16384 + args.prompt, arch.hidden_size)
        dev = tp.device
    else:
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
    model = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0)
    # requests admitted early keep decoding while the rest is prefilled: give every request enough
    # budget to still be running in the timed region
    prefill_steps = (args.batch * args.prompt + 16383) // 16384 + 1
    budget = prefill_steps + args.warmup + args.steps + 4
    total = args.prompt + budget + 2
    pages = args.batch * ((total + 15) // 16 + 1) + 64
    eng = Engine(model, num_pages=pages, page_size=16, max_running=args.batch, max_prefill_tokens=16384,
                 enable_prefix_cache=False, use_cuda_graphs=not args.no_graphs, max_model_len=total + 16,
                 weight_dtype="fp8" if args.fp8 else "bf16", tp=tp)
    if tp is not None and tp.rank != 0:
        eng.follow()
        tp.close()
        return
    g = torch.Generator().manual_seed(0)
    params = SamplingParams(temperature=1.0, max_tokens=budget)
    for _ in range(args.batch):
        eng.submit(Request(prompt=torch.randint(0, arch.vocab_size, (args.prompt,), generator=g).tolist(), params=params))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while eng.waiting or eng._inbox:
        eng.step()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    n0 = eng.stats["generation_tokens"]
    t0 = time.perf_counter()
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    toks = eng.stats["generation_tokens"] - n0
    from ..ops import _runtime as rt

    rt.check_status()
    print(json.dumps({"metric": "rollout decode tokens/s", "model": args.model, "layers": arch.num_hidden_layers,
                      "batch": args.batch, "mean_running": toks / args.steps, "prompt_len": args.prompt, "steps": args.steps,
                      "decode_tokens_per_s": toks / dt, "ms_per_step": 1e3 * dt / args.steps,
                      "prefill_tokens_per_s": args.batch * args.prompt / t_prefill,
                      "peak_memory_gib": torch.cuda.max_memory_allocated() / 2**30, "n_gpus": world,
                      "parallelism": f"tp{world}" if world > 1 else "single", "dtype": "fp8 weights / bf16 KV" if args.fp8 else "bf16", "cuda_graphs": not args.no_graphs,
                      "data": "synthetic (uniform random token ids, random-init weights)"}), flush=True)
    if tp is not None:
        eng.shutdown()
        tp.close()


if __name__ == "__main__":
    main()
