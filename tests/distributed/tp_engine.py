"""Tensor-parallel engine check (child processes, one per GPU or gloo rank):

    python -m torch.distributed.run --nproc-per-node R --master-addr 127.0.0.1 -m tests.distributed.tp_engine

The same prompts through an unsharded engine and through the tensor-parallel one must give the same
greedy tokens; ``--bench-reduce`` first times the fused all-reduce + residual + RMSNorm kernel against
NCCL all-reduce + norm kernel.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from prime_rl_b200.engine.tp import CollectiveTPContext, TPContext, init_tp


def bench_reduce(tp: "TPContext", rows: int = 256, iters: int = 200) -> dict:
    """Device time per call (CUDA events, max over ranks) of the fused reduce and of the same work as
    NCCL all-reduce + fused add-RMSNorm kernel."""
    from prime_rl_b200 import ops

    dev, H = tp.device, tp.hidden
    part = torch.randn(rows, H, device=dev).bfloat16()
    res = torch.randn(rows, H, device=dev).bfloat16()
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)

    def fused():
        tp.reduce(part, res, w, 1e-6)

    def library():
        t = part.clone()
        dist.all_reduce(t, group=tp.group)
        ops.add_rms_norm(t, res, w, 1e-6)

    out = {}
    for name, fn in (("fused", fused), ("nccl", library)):
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        dist.barrier(group=tp.group)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) * 1e3 / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=tp.group)
        out[name] = float(t)
    return out


def selftest(argv=None) -> None:
    """``torchrun --nproc-per-node R -m tests.distributed.tp_engine``: the same prompts through an unsharded
    engine and through the tensor-parallel one must give the same greedy tokens (and close
    log-probabilities); on GPUs the decode step of both is timed."""
    import argparse
    import os
    import time

    from prime_rl_b200.models import ModelArch, build_model, resolve_arch
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.engine.sampler import SamplingParams

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=48)
    ap.add_argument("--tokens", type=int, default=12)
    ap.add_argument("--cuda-graphs", action="store_true")
    ap.add_argument("--weight-dtype", default="bf16")
    ap.add_argument("--skip-reference", action="store_true", help="no unsharded engine (model too large for the check)")
    ap.add_argument("--bench-reduce", action="store_true", help="time the fused reduce against NCCL + norm first")
    ap.add_argument("--prefill-tokens", type=int, default=16384, help="token budget of one prefill step")
    ap.add_argument("--expert-parallel", action="store_true", help="split the experts by index instead of by width")
    args = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    if args.model:
        arch = resolve_arch(args.model)
    else:
        arch = ModelArch(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=3, num_attention_heads=8,
                         num_key_value_heads=4, head_dim=128 if cuda else 32, intermediate_size=512, num_experts=8,
                         num_experts_per_tok=2, moe_intermediate_size=256, vocab_size=2048)
    max_len = args.prompt + args.tokens + 16
    if cuda:
        tp = init_tp(max(max_len, min(args.batch * args.prompt, args.prefill_tokens)), arch.hidden_size)
        dev, dtype = tp.device, torch.bfloat16
    else:
        import datetime

        dist.init_process_group("gloo", timeout=datetime.timedelta(minutes=10))
        dev, dtype = torch.device("cpu"), torch.float32
        tp = CollectiveTPContext(dist.group.WORLD, dev, arch.hidden_size, 1 << 20)
    rank = tp.rank
    if cuda and args.bench_reduce:
        for rows in (8, 256, 4096):
            if rows <= tp.max_tokens:
                r = bench_reduce(tp, rows)
                if rank == 0:
                    print(f"TP_REDUCE rows={rows} cols={arch.hidden_size} fused_us={r['fused']:.1f} "
                          f"nccl_plus_norm_us={r['nccl']:.1f}", flush=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, arch.vocab_size, (args.prompt - (i % 3),), generator=g).tolist() for i in range(args.batch)]
    params = SamplingParams(max_tokens=args.tokens, temperature=0.0)
    kw = dict(num_pages=max(64, args.batch * (max_len // 16 + 2)), page_size=16, enable_prefix_cache=False,
              max_model_len=max_len, max_prefill_tokens=max(max_len, min(args.batch * args.prompt, args.prefill_tokens)),
              max_running=args.batch,
              use_cuda_graphs=args.cuda_graphs, weight_dtype=args.weight_dtype)

    def instrument(engine):
        """Accumulates the synchronised wall time of the decode steps (prefill steps are left out)."""
        acc = {"ms": 0.0, "steps": 0, "tokens": 0, "mark": None}
        inner = engine._decode

        def decode(reqs):
            if engine.mark != acc["mark"]:                          # a new pass began: forget the warm-up
                acc.update(ms=0.0, steps=0, tokens=0, mark=engine.mark)
            if cuda:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            inner(reqs)
            if cuda:
                torch.cuda.synchronize()
            acc["ms"] += (time.perf_counter() - t0) * 1e3
            acc["steps"] += 1
            acc["tokens"] += len(reqs)

        engine._decode = decode
        return acc

    def timed(engine, run):
        acc = instrument(engine)
        out = run()
        return out, acc

    ref = None
    if not args.skip_reference and rank == 0:
        full = Engine(build_model(arch, device=dev, dtype=dtype, seed=0), **kw)
        full.generate_sync(prompts, params)                         # warm-up (graph capture for this batch size)
        ref, ref_acc = timed(full, lambda: full.generate_sync(prompts, params))
        ref = [(r.output, r.logprobs) for r in ref]
        del full
        if cuda:
            torch.cuda.empty_cache()
    dist.barrier()
    eng = Engine(build_model(arch, device=dev, dtype=dtype, seed=0), tp=tp, expert_parallel=args.expert_parallel, **kw)
    if args.expert_parallel and tp.size > 1:
        moe = [l.mlp for l in eng.model.model.layers if getattr(l, "is_moe", False)]
        assert moe and all(m.expert_range == (rank * arch.num_experts // tp.size, (rank + 1) * arch.num_experts // tp.size)
                           and m.experts.gate_up_proj.shape[0] == arch.num_experts // tp.size
                           and m.experts.gate_up_proj.shape[1] == 2 * arch.moe_intermediate_size for m in moe)
    acc = instrument(eng)
    if rank == 0:
        eng.generate_sync(prompts, params)                          # warm-up (graph capture for every batch size)
        if tp.size > 1:
            eng._commands.append(("mark", "timed"))                 # all ranks restart their clocks at the same step
        else:
            eng.mark = "timed"
        out = eng.generate_sync(prompts, params)
        eng.shutdown()
    else:
        eng.follow()
    # a step is as slow as its slowest rank
    worst = torch.tensor([acc["ms"] / max(1, acc["steps"])], dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX, group=tp.control)
    ms = float(worst)
    if cuda:
        from prime_rl_b200.ops import _runtime as rt

        torch.cuda.synchronize()
        rt.check_status()
    ok = True
    if rank == 0:
        if ref is not None:
            same = sum(r.output == o for r, (o, _) in zip(out, ref))
            worst = max((abs(a - b) for r, (_, lp) in zip(out, ref) for a, b in zip(r.logprobs[:1], lp[:1])), default=0.0)
            # bf16 sums in another order can flip a near-tie of the arg-max: most sequences must agree fully,
            # and the first token's log-probability (same context on both sides) must agree closely
            # (random weights give flat distributions: more ranks, more reordered sums, more flipped ties)
            ok = same >= (len(out) if not cuda else len(out) // 2) and worst < (1e-4 if not cuda else 0.08)
            ref_ms = ref_acc["ms"] / max(1, ref_acc["steps"])
            print(f"TP_SELFTEST ranks={tp.size} identical_sequences={same}/{len(out)} first_logprob_diff={worst:.2e} "
                  f"decode_ms_per_step tp={ms:.3f} single={ref_ms:.3f}", flush=True)
        else:
            per = acc["tokens"] / max(1, acc["steps"])
            print(f"TP_SELFTEST ranks={tp.size} decode_ms_per_step tp={ms:.3f} mean_batch={per:.1f} "
                  f"decode_tokens_per_s={per / ms * 1e3:.0f}", flush=True)
        print("TP_SELFTEST_OK" if ok else "TP_SELFTEST_FAIL", flush=True)
    dist.barrier()
    tp.close()
    dist.destroy_process_group()
    if not ok:
        raise SystemExit(1)


if __name__ == "__main__":
    selftest()
