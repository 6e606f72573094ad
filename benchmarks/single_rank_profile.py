"""Runs the peer-memory kernels with a process group of ONE rank (every "peer" pointer is this
GPU's own buffer), so that a single-GPU profiler capture can look at them:

    python -m benchmarks.single_rank_profile --op ep      # dispatch / combine kernels
    python -m benchmarks.single_rank_profile --op rs      # GEMM with the reduce-scatter epilogue
    python -m benchmarks.single_rank_profile --op push    # weight copy / fp8 quantising push
    python -m benchmarks.single_rank_profile --op ep8     # EP dispatch with the fp8 payload
    python -m benchmarks.single_rank_profile --op ag      # GEMM with the all-gather prologue (2 emulated ranks)
    python -m benchmarks.single_rank_profile --op cp      # flash forward with the K/V gather warp (2 emulated ranks)
    python -m benchmarks.single_rank_profile --op zero    # optimizer reduce-scatter pull / all-gather push
    python -m benchmarks.single_rank_profile --op tp      # engine all-reduce + residual + RMSNorm (2 emulated ranks)

The traffic that would cross NVLink stays in local HBM here; instruction mix, occupancy and
local-memory behaviour are what such a capture shows.
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", required=True, choices=["ep", "ep8", "rs", "push", "ag", "cp", "zero", "tp"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=2)
    args = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    group = dist.group.WORLD
    torch.manual_seed(0)
    from prime_rl_b200.ops import _runtime as rt

    if args.op == "ag":
        import ctypes

        M, N, K, rows = args.tokens, 4096, 2048, 2048             # "rank 0" of 2: half of the weight rows are remote
        x = torch.randn(M, K, device=dev).bfloat16()
        mine = torch.randn(N, K, device=dev).bfloat16()
        other = torch.randn(N, K, device=dev).bfloat16()
        ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
        ready = torch.zeros(N // 256, dtype=torch.int32, device=dev)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        for it in range(args.iters):
            rt.check(rt.lib().prb_gemm_bf16_allgather(x.data_ptr(), mine.data_ptr(), ptrs, out.data_ptr(), M, N, K, K, N, 0,
                                                      0, 1.0, 0, 2, rows, ready.data_ptr(), it + 1,
                                                      rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)),
                     "prb_gemm_bf16_allgather")
    elif args.op == "cp":
        import ctypes

        from prime_rl_b200.ops import flash_native

        Tl, Hq, Hkv = args.tokens, 32, 4                          # "rank 1" of 2: chunk 0 is pulled from the other buffer
        T = 2 * Tl
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        q = torch.randn(Tl, Hq, 128, device=dev).bfloat16()
        bufs = [torch.randn(2, T, Hkv, 128, device=dev).bfloat16() for _ in range(2)]
        ptrs = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
        counters = torch.zeros(3, dtype=torch.int32, device=dev)
        for _ in range(args.iters):
            flash_native.flash_fwd_gather(q, bufs[1][0], bufs[1][1], ptrs, cu, 1, 2, counters)
    elif args.op == "tp":
        import ctypes

        rows, cols = args.tokens, 2048                            # "rank 0" of 2; the peer's flag slot is set beforehand
        parts = [torch.randn(rows, cols, device=dev).bfloat16() for _ in range(2)]
        res = torch.randn(rows, cols, device=dev).bfloat16()
        w = torch.ones(cols, dtype=torch.bfloat16, device=dev)
        flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
        flags[0][1] = 1 << 30
        pp = (ctypes.c_void_p * 2)(*[p.data_ptr() for p in parts])
        fp = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
        state = torch.zeros(2, dtype=torch.int32, device=dev)
        out_h, out_x = torch.empty_like(res), torch.empty_like(res)
        for _ in range(args.iters):
            rt.check(rt.lib().prb_ar_add_rmsnorm(pp, fp, state.data_ptr(), res.data_ptr(), w.data_ptr(), out_h.data_ptr(),
                                                 out_x.data_ptr(), rows, cols, 1e-6, 0, 2, rt.status_tensor(dev).data_ptr(),
                                                 rt.stream_ptr(dev)), "prb_ar_add_rmsnorm")
    elif args.op == "zero":
        import ctypes

        n = args.tokens * 16384                                   # 256 MiB of fp32 gradients at the default size
        grads = [torch.randn(n, device=dev) for _ in range(2)]
        flats = [torch.empty(n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        pg = (ctypes.c_void_p * 2)(*[g.data_ptr() for g in grads])
        pf = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flats])
        shard = torch.empty(n // 2, dtype=torch.float32, device=dev)
        for _ in range(args.iters):
            rt.check(rt.lib().prb_rs_pull(pg, 0, n // 2, 0.5, shard.data_ptr(), 2, rt.stream_ptr(dev)), "prb_rs_pull")
            rt.check(rt.lib().prb_ag_push(flats[0].data_ptr(), pf, 0, n, 0, 2, rt.stream_ptr(dev)), "prb_ag_push")
    elif args.op in ("ep", "ep8"):
        from prime_rl_b200.models.layers import GroupedExperts
        from prime_rl_b200.ops import moe as moe_ops
        from prime_rl_b200.parallel.ep_p2p import P2PDispatcher
        from prime_rl_b200.models.config import PRESETS, ModelArch

        def _arch(E, H, I, k):
            return ModelArch(**{**PRESETS["tiny-qwen3-moe"], "num_experts": E, "hidden_size": H,
                                "moe_intermediate_size": I, "num_experts_per_tok": k})

        T, E, H, I, k = args.tokens, 128, 2048, 768, 8
        ex = GroupedExperts(_arch(E, H, I, k), num_local_experts=E, dtype=torch.bfloat16, device=dev)
        with torch.no_grad():
            ex.gate_up_proj.normal_(0, 0.05)
            ex.down_proj.normal_(0, 0.05)
        disp = P2PDispatcher(group, 1, E, capacity_factor=1.0, max_tokens=T, payload="fp8" if args.op == "ep8" else "bf16")
        for _ in range(args.iters):
            x = torch.randn(T, H, device=dev).bfloat16().requires_grad_()
            idx, w, counts = moe_ops.route_topk(torch.randn(T, E, device=dev), k)
            w = w.detach().requires_grad_()
            y = disp(ex, x, idx.to(torch.int32).contiguous(), w, counts)
            y.backward(torch.randn_like(y))
    elif args.op == "rs":
        from prime_rl_b200.parallel.fused_collectives import GemmReduceScatter

        T, N, K = args.tokens, 4096, 2048
        op = GemmReduceScatter(group, N, K, dev)
        dy, x = torch.randn(T, N, device=dev).bfloat16(), torch.randn(T, K, device=dev).bfloat16()
        for _ in range(args.iters):
            op(dy, x, a_mn=True, b_mn=True)
    else:
        from prime_rl_b200.models.fp8 import quantize_to_fp8_blockwise

        w = torch.randn(args.tokens * 16, 2048, device=dev).bfloat16()       # 256 MB at the default size
        dst = torch.empty_like(w)
        for _ in range(args.iters):
            rt.check(rt.lib().prb_weight_push(w.data_ptr(), dst.data_ptr(), w.numel() * 2, rt.stream_ptr(dev)),
                     "prb_weight_push")
            quantize_to_fp8_blockwise(w)
    torch.cuda.synchronize()
    rt.check_status()
    print("SINGLE_RANK_PROFILE_OK", args.op, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
