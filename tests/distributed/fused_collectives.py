"""GEMM -> reduce-scatter and all-gather -> GEMM over peer memory against "GEMM + NCCL collective"
(child processes, one per GPU):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m tests.distributed.fused_collectives

Prints FUSED_RS_OK / FUSED_AG_OK; with FUSED_SELFTEST_TIMING=1 also device times (CUDA events, max over ranks).
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.parallel.fused_collectives import AllGatherGemm, GemmReduceScatter


def _selftest_allgather(group, dev, rank, world) -> bool:
    from prime_rl_b200.ops.matmul import gemm

    torch.manual_seed(11)
    N, K, M = 256 * world * 2, 520, 1000
    w_full = (torch.randn(N, K, device=dev) * 0.05).bfloat16()          # same on every rank (same seed)
    x = torch.randn(M, K, device=dev).bfloat16()
    op = AllGatherGemm(group, N, K, dev)
    worst = 0.0
    for it in range(2):                                                   # second call: counters keep growing
        op.weight.fill_(float("nan"))
        op.shard.copy_(w_full[rank * op.rows:(rank + 1) * op.rows] * (it + 1))
        y = op(x)
        ref = x.float() @ (w_full.float() * (it + 1)).t()
        torch.cuda.synchronize()
        rt.check_status()
        worst = max(worst, float((y.float() - ref).abs().max() / ref.abs().max()))
        if not torch.equal(op.weight, w_full * (it + 1)):
            worst = float("inf")
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 2e-2
    if rank == 0:
        print(("FUSED_AG_OK" if ok else "FUSED_AG_FAIL"), "max relative deviation", float(t), flush=True)
    op.close()
    if ok and os.environ.get("FUSED_SELFTEST_TIMING", "1") == "1":
        M, N, K = 16384, 4096, 2048
        x = torch.randn(M, K, device=dev).bfloat16()
        op = AllGatherGemm(group, N, K, dev)
        op.shard.normal_(std=0.02)
        gathered = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

        def base():
            dist.all_gather_into_tensor(gathered, op.shard, group=group)
            gemm(x, gathered, out=out)

        for name, fn in (("NCCL all_gather + GEMM", base),
                         ("fused (gather warps inside the GEMM)", lambda: op(x, out=out))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(10):
                fn()
            e.record()
            torch.cuda.synchronize()
            rt.check_status()
            ms = torch.tensor([s.elapsed_time(e) / 10], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                flops = 2 * M * N * K
                print(f"FUSED_AG_TIMING {name}: {float(ms):.3f} ms ({flops / float(ms) / 1e9:.0f} TFLOP/s per GPU; "
                      f"weight {N}x{K} bf16 over {world} ranks, max over ranks)", flush=True)
        op.close()
    return ok


def _selftest() -> int:
    """python -m torch.distributed.run --nproc-per-node N -m tests.distributed.fused_collectives"""
    import os
    import sys

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    torch.manual_seed(7 + rank)
    ok = True
    # numerics: weight-gradient form (A, B MN-major), ragged sizes
    T, Nout, Kin = 1000, 384, 520
    dy = torch.randn(T, Nout, device=dev).bfloat16()
    x = torch.randn(T, Kin, device=dev).bfloat16()
    op = GemmReduceScatter(group, Nout, Kin, dev)
    got = op(dy, x, a_mn=True, b_mn=True).clone()
    got2 = op(dy, x, a_mn=True, b_mn=True, accumulate=True).clone()
    full = dy.float().t() @ x.float()
    dist.all_reduce(full)
    rows = op.rows
    ref = full[rank * rows:(rank + 1) * rows]
    torch.cuda.synchronize()
    rt.check_status()
    e1 = float((got[:ref.shape[0]] - ref).abs().max() / ref.abs().max())
    e2 = float((got2[:ref.shape[0]] - 2 * ref).abs().max() / ref.abs().max())
    t = torch.tensor([max(e1, e2)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 2e-2
    if rank == 0:
        print(("FUSED_RS_OK" if ok else "FUSED_RS_FAIL"), "max relative deviation", float(t), flush=True)
    op.close()
    if ok and os.environ.get("FUSED_SELFTEST_TIMING", "1") == "1":
        # timing: weight gradient of a 16384-token micro-batch, [4096 x 2048], against GEMM + NCCL
        T, Nout, Kin = 16384, 4096, 2048
        dy = torch.randn(T, Nout, device=dev).bfloat16()
        x = torch.randn(T, Kin, device=dev).bfloat16()
        op = GemmReduceScatter(group, Nout, Kin, dev)
        from prime_rl_b200.ops.matmul import gemm

        full = torch.empty(Nout, Kin, dtype=torch.float32, device=dev)
        shard = torch.empty(Nout // world, Kin, dtype=torch.float32, device=dev)

        def base():
            gemm(dy, x, a_mn=True, b_mn=True, out=full)
            dist.reduce_scatter_tensor(shard, full, group=group)

        for name, fn in (("GEMM + NCCL reduce_scatter", base),
                         ("fused (peer reductions in the epilogue)", lambda: op(dy, x, a_mn=True, b_mn=True))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(10):
                fn()
            e.record()
            torch.cuda.synchronize()
            rt.check_status()
            ms = torch.tensor([s.elapsed_time(e) / 10], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                flops = 2 * T * Nout * Kin
                print(f"FUSED_RS_TIMING {name}: {float(ms):.3f} ms ({flops / float(ms) / 1e9:.0f} TFLOP/s per GPU; "
                      f"{Nout}x{Kin} fp32 over {world} ranks, max over ranks)", flush=True)
        op.close()
    ok = _selftest_allgather(group, dev, rank, world) and ok
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    import sys

    sys.exit(_selftest())
