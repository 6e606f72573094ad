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
