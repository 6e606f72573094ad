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


def run_rollout_bench(model: str = "qwen3-30b-a3b", contexts=(1024, 3072, 5120), steps: int = 16, warmup: int = 3,
                      layers: int | None = None, dev: torch.device | None = None, prompts: int = 32, samples: int = 8,
                      prompt_len: int = 1024, fp8: bool = True, max_tp: int = 4, graphs: bool = True,
                      prefix_splits: int | None = None) -> dict | None:
    """The rollout half of the headline benchmark. Collective: every rank of the launch calls it; rank 0
    gets the result, the others ``None``.

    ``prompts x samples`` concurrent requests per engine group; the samples of a prompt share its pages
    through the prefix cache. Tensor parallelism over ``min(world, kv heads, max_tp)`` GPUs, data-parallel
    groups beyond that (tokens/s summed over the groups, step time = the slowest group). For every context
    length C the requests are brought to a KV length of C (the shared prompt plus C - prompt_len tokens of
    their own, entered as a prefill: a decode step costs the same whether the cache was filled by decoding
    or by prefill) and ``steps`` decode steps through ``Engine.step`` are timed on the device clock of the
    group's rank 0, each ending with the device-to-host read of the sampled tokens. Then every rank times one
    full weight update bf16 -> fp8 in flight into a peer's live fp8 buffers (``csrc/weight_push.cu``)."""
    import torch.distributed as dist

    from .tp import TPContext

    arch = resolve_arch(model)
    if layers:
        arch = arch.model_copy(update={"num_hidden_layers": layers})
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if dev is None:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    tp_size = 1
    while tp_size * 2 <= min(world, arch.num_key_value_heads, max_tp) and world % (tp_size * 2) == 0:
        tp_size *= 2
    groups = world // tp_size
    batch = prompts * samples
    c_max = max(contexts)
    prefill_budget = 16384

    def decode_budget(C: int) -> int:
        # requests admitted early keep decoding while the rest is prefilled: every request must still be
        # running when the timed steps end
        prefill_tokens = prompts * C + (batch - prompts) * (C - prompt_len)
        return (prefill_tokens + prefill_budget - 1) // prefill_budget + prompts + warmup + steps + 8

    budget = decode_budget(c_max)
    max_len = c_max + budget + 16
    tp = None
    if tp_size > 1:
        import datetime

        mine = None
        for g in range(groups):            # every rank creates every group, in the same order
            ranks = list(range(g * tp_size, (g + 1) * tp_size))
            data = dist.new_group(ranks=ranks)
            ctrl = dist.new_group(ranks=ranks, backend="gloo", timeout=datetime.timedelta(hours=2))
            if rank in ranks:
                mine = (data, ctrl)
        tp = TPContext(mine[0], dev, arch.hidden_size, max(prefill_budget, max_len), control_group=mine[1])
    net = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0)
    # pages: every request's own tokens plus one shared prompt per group of samples, plus slack
    own_pages = (c_max - prompt_len + budget + 15) // 16 + 2
    pages = batch * own_pages + prompts * (prompt_len // 16 + 1) + 256
    eng = Engine(net, num_pages=pages, page_size=16, max_running=batch, max_prefill_tokens=prefill_budget,
                 enable_prefix_cache=True, use_cuda_graphs=graphs, max_model_len=max_len,
                 weight_dtype="fp8" if fp8 else "bf16", tp=tp, keep_bf16_weights=not fp8)
    if prefix_splits:
        eng.runner.prefix_splits = int(prefix_splits)       # before the first decode graph is captured
    leader = tp is None or tp.rank == 0
    points = []
    failure = None

    def drive():
        g = torch.Generator().manual_seed(1234 + rank)
        for C in contexts:
            params = SamplingParams(temperature=1.0, max_tokens=decode_budget(C))
            shared = [torch.randint(0, arch.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(prompts)]

            def tail():
                return torch.randint(0, arch.vocab_size, (C - prompt_len,), generator=g).tolist() if C > prompt_len else []

            # the first sample of every prompt fills (and registers) the shared pages ...
            first = [eng.submit(Request(prompt=p + tail(), params=params)) for p in shared]
            while eng.waiting or eng._inbox:
                eng.step()
            hits0 = eng.stats["prefix_hits"]
            # ... the other samples find them in the prefix cache
            rest = [eng.submit(Request(prompt=p + tail(), params=params)) for p in shared for _ in range(samples - 1)]
            while eng.waiting or eng._inbox:
                eng.step()
            shared_tokens = eng.stats["prefix_hits"] - hits0
            for _ in range(warmup):
                eng.step()
            torch.cuda.synchronize()
            running = len(eng.running)
            n0 = eng.stats["generation_tokens"]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            toks = eng.stats["generation_tokens"] - n0
            if running < batch:
                raise RuntimeError(f"only {running} of {batch} requests were running at context {C}: the KV pool is too "
                                   "small for the benchmark (requests were preempted)")
            points.append({"context": C, "ms_per_step": e0.elapsed_time(e1) / steps, "wall_ms_per_step": 1e3 * wall / steps,
                           "tokens": toks, "running": running, "prefix_shared_tokens": shared_tokens,
                           "kv_usage": eng.cache.blocks.usage})
            while eng.running or eng.waiting:           # let the requests run out before the next context
                eng.step()
            del first, rest
            eng.clear_prefix_cache()                    # the next context needs the pages these prompts still hold
            if tp is not None:
                eng.step()                              # carries the command to the other ranks
        from ..ops import _runtime as rt

        rt.check_status()

    if not leader:
        eng.follow()
    else:
        try:
            drive()
        except Exception as e:      # the other ranks of the group wait in follow(): release them whatever happened
            failure = f"{type(e).__name__}: {e}"[:300]
        finally:
            if tp is not None:
                eng.shutdown()
    # ---------------------------------------------------------------- one weight update, quantised in flight
    push = _timed_weight_push(eng, dev, world, rank) if fp8 else None
    # ---------------------------------------------------------------- merge over the groups
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    local = {"points": points, "push": push, "mem": mem, "leader": leader, "failure": failure}
    gathered = [local]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, local)
    if tp is not None:
        tp.close()
    failures = [x["failure"] for x in gathered if x.get("failure")]
    if failures:
        raise RuntimeError(f"rollout benchmark failed on {len(failures)} engine group(s): {failures[0]}")
    if rank != 0:
        return None
    leaders = [x for x in gathered if x["leader"]]
    out_points = []
    for i, C in enumerate(contexts):
        ms = max(x["points"][i]["ms_per_step"] for x in leaders)
        toks = sum(x["points"][i]["tokens"] for x in leaders)
        out_points.append({"context": C, "ms_per_step": ms, "tokens_per_s": toks / steps / ms * 1e3,
                           "running_per_group": leaders[0]["points"][i]["running"],
                           "prefix_shared_tokens_per_group": leaders[0]["points"][i]["prefix_shared_tokens"],
                           "kv_usage": leaders[0]["points"][i]["kv_usage"]})
    mean_ms = sum(p["ms_per_step"] for p in out_points) / len(out_points)
    res = {"metric": "rollout decode tokens/s", "value": sum(p["tokens_per_s"] for p in out_points) / len(out_points),
           "unit": "tokens/s", "ms_per_step": mean_ms, "by_context": out_points,
           "requests_per_group": batch, "samples_per_prompt": samples, "prompt_len": prompt_len,
           "generated_len": c_max - prompt_len, "steps_per_context": steps,
           "parallelism": f"tp{tp_size} x dp{groups}", "cuda_graphs": True, "page_size": 16,
           "dtype": "fp8 weights (128x128 blocks, 1x128 activation scales), bf16 KV" if fp8 else "bf16",
           "peak_memory_gib": max(x["mem"] for x in gathered)}
    if push is not None:
        pushes = [x["push"] for x in gathered if x["push"]]
        res["weight_sync"] = {"ms": max(p["ms"] for p in pushes), "source_gb_per_gpu": pushes[0]["source_gb"],
                              "gb_per_s_per_gpu": min(p["gb_per_s"] for p in pushes), "target": pushes[0]["target"],
                              "note": pushes[0]["note"]}
    return res


def _timed_weight_push(eng, dev, world: int, rank: int) -> dict:
    """Every rank pushes new bf16 values for a whole engine shard into the live fp8 buffers of the next
    rank's engine (its own when there is one GPU), quantising to e4m3 + 128 x 128 scales on the way."""
    import torch.distributed as dist

    from ..transports.weights.p2p import P2PWeightPort, _Mapped, push_state

    port = P2PWeightPort(eng.model, None, replica=rank, quantize="fp8")
    manifests = [port.manifest]
    if world > 1:
        manifests = [None] * world
        dist.all_gather_object(manifests, port.manifest)
    target = manifests[(rank + 1) % world]
    mapped = _Mapped() if world > 1 else None

    # source values: the bf16 copy was released, so one buffer per distinct shape stands in for the trainer's
    # shard (its contents do not matter for the timing; it is far larger than L2 in total)
    sources: dict[tuple, torch.Tensor] = {}
    tensors = {}
    for name, e in target["params"].items():
        key = (tuple(e["shape"]), e["dtype"])
        if key not in sources:
            sources[key] = (torch.randn(e["shape"], device=dev, dtype=torch.bfloat16) * 0.02).to(
                getattr(torch, e["dtype"]))
        tensors[name] = sources[key]
    src_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
    if world > 1:
        dist.barrier()
        resolver = mapped
    else:
        resolver = _SelfResolver(port)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    push_state(tensors, target, resolver)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        mapped.close()
    return {"ms": ms, "source_gb": src_bytes / 1e9, "gb_per_s": src_bytes / ms / 1e6,
            "target": "next rank's engine over NVLink" if world > 1 else "same GPU",
            "note": "bf16 source values of one engine shard -> e4m3 + 128x128 fp32 scales written into the live "
                    "fp8 buffers; one source buffer per distinct tensor shape"}


class _SelfResolver:
    """Resolves manifest entries of this process's own port to local device pointers (no IPC mapping)."""

    def __init__(self, port):
        self.by_handle = {}
        for name, e in port.manifest["params"].items():
            if "fp8" in e:
                q, s = port.live_fp8.get(name) or port.fp8[name]
                self.by_handle[(e["fp8"]["q"]["handle"], e["fp8"]["q"]["offset"])] = q.data_ptr()
                self.by_handle[(e["fp8"]["scales"]["handle"], e["fp8"]["scales"]["offset"])] = s.data_ptr()
            if "handle" in e:
                self.by_handle[(e["handle"], e["offset"])] = port.params[name].data_ptr()

    def ptr(self, entry: dict) -> int:
        return self.by_handle[(entry["handle"], entry["offset"])]


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
    ap.add_argument("--rollout", action="store_true",
                    help="the shared-prefix rollout measurement (32 prompts x 8 samples) instead of independent prompts")
    ap.add_argument("--contexts", default="1024,3072,5120", help="--rollout: KV lengths at which decode steps are timed")
    ap.add_argument("--prefix-splits", type=int, default=None,
                    help="--rollout: slices of a group's shared pages handled by different CTAs (default: the runner's)")
    args = ap.parse_args(argv)
    if args.rollout:
        res = run_rollout_bench(args.model, [int(c) for c in args.contexts.split(",")], args.steps, args.warmup,
                                args.layers, fp8=args.fp8, graphs=not args.no_graphs, prefix_splits=args.prefix_splits)
        if res is not None:
            print(json.dumps(res), flush=True)
        return
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
