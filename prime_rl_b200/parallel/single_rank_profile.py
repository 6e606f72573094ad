"""Runs the peer-memory kernels with a process group of ONE rank (every "peer" pointer is this
GPU's own buffer), so that a single-GPU profiler capture can look at them:

    python -m prime_rl_b200.parallel.single_rank_profile --op ep      # dispatch / combine kernels
    python -m prime_rl_b200.parallel.single_rank_profile --op rs      # GEMM with the reduce-scatter epilogue
    python -m prime_rl_b200.parallel.single_rank_profile --op push    # weight copy / fp8 quantising push

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
    ap.add_argument("--op", required=True, choices=["ep", "rs", "push"])
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
    from ..ops import _runtime as rt

    if args.op == "ep":
        from ..models.layers import GroupedExperts
        from ..ops import moe as moe_ops
        from .ep_p2p import P2PDispatcher
        from .ep_selftest import _arch

        T, E, H, I, k = args.tokens, 128, 2048, 768, 8
        ex = GroupedExperts(_arch(E, H, I, k), num_local_experts=E, dtype=torch.bfloat16, device=dev)
        with torch.no_grad():
            ex.gate_up_proj.normal_(0, 0.05)
            ex.down_proj.normal_(0, 0.05)
        disp = P2PDispatcher(group, 1, E, capacity_factor=1.0, max_tokens=T)
        for _ in range(args.iters):
            x = torch.randn(T, H, device=dev).bfloat16().requires_grad_()
            idx, w, counts = moe_ops.route_topk(torch.randn(T, E, device=dev), k)
            w = w.detach().requires_grad_()
            y = disp(ex, x, idx.to(torch.int32).contiguous(), w, counts)
            y.backward(torch.randn_like(y))
    elif args.op == "rs":
        from .fused_collectives import GemmReduceScatter

        T, N, K = args.tokens, 4096, 2048
        op = GemmReduceScatter(group, N, K, dev)
        dy, x = torch.randn(T, N, device=dev).bfloat16(), torch.randn(T, K, device=dev).bfloat16()
        for _ in range(args.iters):
            op(dy, x, a_mn=True, b_mn=True)
    else:
        from ..models.fp8 import quantize_to_fp8_blockwise

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
