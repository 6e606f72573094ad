"""GEMMs fused with their collective over NVLink peer memory: GEMM -> reduce-scatter and
all-gather -> GEMM.

``GemmReduceScatter`` computes ``C = alpha * A.B`` on every rank (each rank holds its own A / B,
e.g. its micro-batch's activations and output gradients for a weight gradient, or its K-slice
of a row-parallel linear) and leaves ``sum_over_ranks(C)[rows of rank r]`` on rank r. The tile
leaves TMEM as fp32 vector reductions into the owner's shard (``csrc/gemm.cu: EpiPeerReduce``),
so the NVLink traffic of one tile overlaps the tensor-core work of the next and the full partial
product never exists in memory. A stream-ordered flag exchange (``csrc/ep_p2p.cu``) brackets
the kernel: shards are zeroed before anybody adds, and complete before anybody reads.

``AllGatherGemm`` computes ``y = x W^T`` for a weight whose rows are sharded over the ranks
(the layout FSDP keeps parameters in). Every rank holds a full-size buffer of which its own rows
are valid; two extra warps per CTA of the GEMM kernel copy the other ranks' rows over NVLink
into that buffer (``csrc/gemm.cu: SchedAllGather / ag_gather``) while the tensor cores already
work on the N blocks of the local rows, and the TMA producer waits on a per-N-block arrival
counter before it loads a remote block. After the call the buffer holds the whole weight, so the
backward GEMMs can use it without a second gather. Takes the place of the reference's FSDP2
parameter all-gather followed by the first GEMM of the unit (src/prime_rl/trainer/model.py:470-559).

``GemmReduceScatter`` takes the place of "GEMM, then ``reduce_scatter_tensor``" (the reference's FSDP2 gradient
reduce-scatter, src/prime_rl/trainer/parallel_dims.py / torch FSDP; vLLM's row-parallel
all-reduce in the engine).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _runtime as rt
from .symm import SymmetricBuffer

_K_ZEROED, _K_DONE = 0, 1


class GemmReduceScatter:
    def __init__(self, group, M: int, N: int, device: torch.device):
        self.group = group
        self.R = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.R > 8:
            raise ValueError("at most 8 ranks (one NVSwitch box)")
        self.M, self.N = M, N
        self.rows = (M + self.R - 1) // self.R
        shard_bytes = self.rows * N * 4
        self.off_flags = (shard_bytes + 255) // 256 * 256
        self.mem = SymmetricBuffer(group, self.off_flags + 256, device, zero=True)
        self.shard = self.mem.local(torch.float32, 0, self.rows * N).view(self.rows, N)
        self.flags = self.mem.local(torch.int32, self.off_flags, 2 * self.R)
        self.p_c = self.mem.offset_ptrs(0)
        self.p_flags = self.mem.offset_ptrs(self.off_flags)
        self.epoch = 0
        self.device = device

    def __call__(self, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
                 alpha: float = 1.0, accumulate: bool = False) -> torch.Tensor:
        """Returns this rank's fp32 shard ``[rows_per_rank, N]`` (a view of the symmetric buffer,
        valid until the next call). ``accumulate`` keeps the previous contents (running sum over
        micro-batches)."""
        lib, dev = rt.lib(), self.device
        M = a.shape[1] if a_mn else a.shape[0]
        K = a.shape[0] if a_mn else a.shape[1]
        N = b.shape[1] if b_mn else b.shape[0]
        assert (M, N) == (self.M, self.N) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        assert a.stride(1) == 1 and b.stride(1) == 1
        self.epoch += 1
        ep, st, stream = self.epoch, rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)
        if not accumulate:
            self.shard.zero_()
        # everybody's shard is ready to receive
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, self.R, _K_ZEROED, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), self.R, _K_ZEROED, ep, st, stream), "prb_ep_wait")
        rt.check(lib.prb_gemm_bf16_reduce_scatter(a.data_ptr(), b.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                                  int(a_mn), int(b_mn), float(alpha), self.p_c, self.R, self.rows,
                                                  N, st, stream), "prb_gemm_bf16_reduce_scatter")
        # my reductions are performed (kernel boundary), tell the owners; then wait for all senders
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, self.R, _K_DONE, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), self.R, _K_DONE, ep, st, stream), "prb_ep_wait")
        return self.shard

    def close(self):
        self.mem.close()


class AllGatherGemm:
    """``y = x W^T`` with ``W [N, K]`` row-sharded over the group (``N / R`` rows per rank, a multiple
    of 256; ``K`` a multiple of 8)."""

    def __init__(self, group, N: int, K: int, device: torch.device):
        self.group = group
        self.R = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.R > 8:
            raise ValueError("at most 8 ranks (one NVSwitch box)")
        if N % (256 * self.R) or K % 8:
            raise ValueError("N must be a multiple of 256 * ranks and K of 8")
        self.N, self.K, self.rows = N, K, N // self.R
        w_bytes = N * K * 2
        self.off_ready = (w_bytes + 255) // 256 * 256
        self.off_flags = self.off_ready + (N // 256 * 4 + 255) // 256 * 256
        self.mem = SymmetricBuffer(group, self.off_flags + 256, device, zero=True)
        self.weight = self.mem.local(torch.bfloat16, 0, N * K).view(N, K)
        self.shard = self.weight[self.rank * self.rows:(self.rank + 1) * self.rows]    # the rows this rank owns
        self.ready = self.mem.local(torch.int32, self.off_ready, N // 256)
        self.flags = self.mem.local(torch.int32, self.off_flags, 2 * self.R)
        self.p_flags = self.mem.offset_ptrs(self.off_flags)
        self.calls = 0
        self.device = device

    def __call__(self, x: torch.Tensor, *, out: torch.Tensor | None = None, alpha: float = 1.0) -> torch.Tensor:
        """``x [M, K]`` bf16 -> ``[M, N]`` bf16. The caller writes ``self.shard`` before the call."""
        lib, dev = rt.lib(), self.device
        M = x.shape[0]
        assert x.dtype == torch.bfloat16 and x.shape[1] == self.K and x.stride(1) == 1
        if out is None:
            out = torch.empty(M, self.N, dtype=torch.bfloat16, device=dev)
        self.calls += 1
        ep, st, stream = self.calls, rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)
        # every rank's rows are written (stream order on the owner), then visible to the readers
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, self.R, _K_ZEROED, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), self.R, _K_ZEROED, ep, st, stream), "prb_ep_wait")
        rt.check(lib.prb_gemm_bf16_allgather(x.data_ptr(), self.weight.data_ptr(), self.mem.c_ptrs, out.data_ptr(),
                                             M, self.N, self.K, x.stride(0), out.stride(0), 0,
                                             int(out.dtype == torch.float32), float(alpha), self.rank, self.R,
                                             self.rows, self.ready.data_ptr(), ep, st, stream),
                 "prb_gemm_bf16_allgather")
        # all readers are done with my rows before I may rewrite them
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, self.R, _K_DONE, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), self.R, _K_DONE, ep, st, stream), "prb_ep_wait")
        return out

    def close(self):
        self.mem.close()


def _selftest_allgather(group, dev, rank, world) -> bool:
    from ..ops.matmul import gemm

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
    """python -m torch.distributed.run --nproc-per-node N -m prime_rl_b200.parallel.fused_collectives"""
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
        from ..ops.matmul import gemm

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
