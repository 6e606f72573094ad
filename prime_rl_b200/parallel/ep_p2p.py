"""Peer-memory expert-parallel dispatcher: tokens are written by the sending GPU straight into
their final row of the owner's expert-sorted buffer and come back through peer loads fused with
the top-k weighted sum (``csrc/ep_p2p.cu``). No host read of split sizes, no staging copy, no
library collective on the data path.

Data flow of one MoE call on every rank (all on the current stream):

    counts ──hist push──▶ all peers      plan: where do my rows of expert e start on its owner?
    x rows ──push──────▶ owners' xbuf    (flag per sender)            ┐ _Dispatch
    wait senders, zero padding rows, experts(xbuf)                     ┘
    y ─▶ ybuf, "ready" flag ─▶ peers     out[t] = Σ_k w · peer_row    ─ _Combine

Backward runs the same two trips in the other direction (gradient rows are pushed scaled by
the routing weight, input gradients are pulled and summed). The four row buffers are reused by
every layer; that is safe because any two uses are separated by a complete flag exchange among
all ranks, and it requires per-layer activation recomputation for training (the tensors autograd
keeps are views of these buffers).

``payload="fp8"`` sends the forward dispatch as e4m3 with one fp32 scale per row and 128 columns
(quantised by the sending warp on its way out, expanded to bf16 by the owner after the flags):
half the NVLink bytes of the largest transfer. The combine and both backward trips stay bf16, as
in the reference's quantised all-to-all (src/prime_rl/trainer/distributed/collectives.py:95-152).

Same role as the reference's DeepEP path (src/prime_rl/trainer/distributed/deepep.py,
token_dispatcher.py:303-420).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _runtime as rt
from ..ops import moe as moe_ops
from ..ops import stash
from .symm import SymmetricBuffer

K_HIST, K_DATA_X, K_OUT_Y, K_DATA_G, K_OUT_DX = range(5)


class _Shared:
    """Symmetric buffers of one (group, hidden size, capacity); shared by all MoE layers."""

    _cache: dict = {}

    def __init__(self, group, R: int, E: int, H: int, cap_rows: int, device, fp8: bool = False):
        self.group, self.R, self.E, self.H, self.cap = group, R, E, H, cap_rows
        self.rank = dist.get_rank(group)
        row_bytes = cap_rows * H * 2
        self.off_x, self.off_y, self.off_g, self.off_dx = 0, row_bytes, 2 * row_bytes, 3 * row_bytes
        self.off_hist = 4 * row_bytes
        self.off_flags = self.off_hist + R * E * 4
        # arrival counters of the per-block dispatch: [parity][128-row block of xbuf]
        self.max_blocks = cap_rows // 128
        self.off_cnt = (self.off_flags + 5 * R * 4 + 15) // 16 * 16
        total = self.off_cnt + 2 * self.max_blocks * 4
        total = (total + 255) // 256 * 256
        self.fp8 = fp8
        if fp8:
            if H % 128:
                raise ValueError("the fp8 payload needs a hidden size that is a multiple of 128")
            self.off_q = total
            self.off_s = self.off_q + cap_rows * H
            total = (self.off_s + cap_rows * (H // 128) * 4 + 255) // 256 * 256
        self.mem = SymmetricBuffer(group, total, device, zero=True)
        m = self.mem
        self.xbuf = m.local(torch.bfloat16, self.off_x, cap_rows * H).view(cap_rows, H)
        self.ybuf = m.local(torch.bfloat16, self.off_y, cap_rows * H).view(cap_rows, H)
        self.gbuf = m.local(torch.bfloat16, self.off_g, cap_rows * H).view(cap_rows, H)
        self.dxbuf = m.local(torch.bfloat16, self.off_dx, cap_rows * H).view(cap_rows, H)
        self.hist = m.local(torch.int32, self.off_hist, R * E).view(R, E)
        self.flags = m.local(torch.int32, self.off_flags, 5 * R)
        self.p_x, self.p_y = m.offset_ptrs(self.off_x), m.offset_ptrs(self.off_y)
        self.p_g, self.p_dx = m.offset_ptrs(self.off_g), m.offset_ptrs(self.off_dx)
        self.p_hist, self.p_flags = m.offset_ptrs(self.off_hist), m.offset_ptrs(self.off_flags)
        self.cnt = m.local(torch.int32, self.off_cnt, 2 * self.max_blocks).view(2, self.max_blocks)
        self.p_cnt = m.offset_ptrs(self.off_cnt)
        self.blk_epoch = 0
        self.side = torch.cuda.Stream(device=device)
        if fp8:
            self.qbuf = m.local(torch.uint8, self.off_q, cap_rows * H).view(cap_rows, H)
            self.sbuf = m.local(torch.float32, self.off_s, cap_rows * (H // 128)).view(cap_rows, H // 128)
            self.p_q, self.p_s = m.offset_ptrs(self.off_q), m.offset_ptrs(self.off_s)
        self.epoch = [0] * 5
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.device = device

    def next_epoch(self, kind: int) -> int:
        self.epoch[kind] += 1
        return self.epoch[kind]

    @classmethod
    def get(cls, group, R, E, H, cap_rows, device, fp8: bool = False):
        key = (id(group), R, E, H, device.index, fp8)
        sh = cls._cache.get(key)
        if sh is None or sh.cap < cap_rows:
            sh = cls(group, R, E, H, cap_rows, device, fp8)
            cls._cache[key] = sh
        return sh


def release_shared() -> None:
    """Frees the symmetric buffers of every dispatcher of this process (collective over their groups)."""
    for sh in list(_Shared._cache.values()):
        sh.mem.close()
    _Shared._cache.clear()


class _Route:
    """Per-call routing state shared by the two autograd functions."""
    __slots__ = ("sh", "idx", "slot", "local_off", "send_base", "pos", "hist", "expert_offset", "block_expert",
                 "T", "k", "ep_y", "local", "counts", "block_rows", "push_done")


def _status(dev):
    return rt.status_tensor(dev).data_ptr()


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, route: _Route, per_block: bool = False):
        sh, lib, dev = route.sh, rt.lib(), x.device
        x = x.contiguous()
        ctx.route = route
        if per_block:
            # no global wait: the owner prepares its buffer, the rows leave on a side stream in the order of the
            # owners' buffers, and the grouped GEMM that follows waits per 128-row block on the arrival counters
            sh.blk_epoch += 1
            par = sh.blk_epoch & 1
            local = route.local
            route.block_rows = torch.empty(sh.max_blocks, dtype=torch.int32, device=dev)
            rt.check(lib.prb_ep_prepare(sh.xbuf.data_ptr(), route.hist.data_ptr(), route.expert_offset.data_ptr(),
                                        route.block_rows.data_ptr(), sh.cnt[1 - par].data_ptr(), sh.max_blocks,
                                        sh.rank, sh.R, sh.E, sh.H, rt.stream_ptr(dev)), "prb_ep_prepare")
            main = torch.cuda.current_stream(dev)
            sh.side.wait_stream(main)
            with torch.cuda.stream(sh.side):
                rt.check(lib.prb_ep_push_blocks(x.data_ptr(), local.row_src.data_ptr(), local.block_expert.data_ptr(),
                                                local.expert_offset.data_ptr(), local.total_rows.data_ptr(),
                                                route.counts.data_ptr(), route.send_base.data_ptr(), sh.p_x, sh.p_cnt,
                                                par * sh.max_blocks * 4, route.pos.data_ptr(),
                                                local.block_expert.numel(), route.k, sh.H, sh.E, sh.rank, sh.R, sh.cap,
                                                _status(dev), rt.stream_ptr(dev)), "prb_ep_push_blocks")
                route.push_done = torch.cuda.Event()
                route.push_done.record(sh.side)
            x.record_stream(sh.side)
            xin = sh.xbuf.view(sh.cap, sh.H)
            xin._blk_ready = (sh.cnt[par], route.block_rows)
            return xin
        ep = sh.next_epoch(K_DATA_X)
        if sh.fp8:
            rt.check(lib.prb_ep_push_fp8(x.data_ptr(), route.idx.data_ptr(), route.slot.data_ptr(),
                                         route.local_off.data_ptr(), route.send_base.data_ptr(), None, None, sh.p_q,
                                         sh.p_s, sh.p_flags, route.pos.data_ptr(), sh.done.data_ptr(),
                                         route.T * route.k, route.k, sh.H, sh.E, sh.rank, sh.R, K_DATA_X, ep, sh.cap,
                                         _status(dev), rt.stream_ptr(dev)), "prb_ep_push_fp8")
            rt.check(lib.prb_ep_recv_fp8(sh.xbuf.data_ptr(), sh.qbuf.data_ptr(), sh.sbuf.data_ptr(),
                                         route.hist.data_ptr(), route.expert_offset.data_ptr(), sh.flags.data_ptr(),
                                         sh.rank, sh.R, sh.E, sh.H, K_DATA_X, ep, _status(dev), rt.stream_ptr(dev)),
                     "prb_ep_recv_fp8")
        else:
            rt.check(lib.prb_ep_push(x.data_ptr(), route.idx.data_ptr(), route.slot.data_ptr(),
                                     route.local_off.data_ptr(), route.send_base.data_ptr(), None, None, sh.p_x,
                                     sh.p_flags, route.pos.data_ptr(), sh.done.data_ptr(), route.T * route.k, route.k,
                                     sh.H, sh.E, sh.rank, sh.R, K_DATA_X, ep, sh.cap, _status(dev),
                                     rt.stream_ptr(dev)), "prb_ep_push")
            rt.check(lib.prb_ep_recv(sh.xbuf.data_ptr(), route.hist.data_ptr(), route.expert_offset.data_ptr(),
                                     sh.flags.data_ptr(), sh.rank, sh.R, sh.E, sh.H, K_DATA_X, ep, _status(dev),
                                     rt.stream_ptr(dev)), "prb_ep_recv")
        xin = sh.xbuf.view(sh.cap, sh.H)         # a fresh tensor object over the shared buffer
        return xin

    @staticmethod
    def backward(ctx, g):
        route = ctx.route
        sh, lib, dev = route.sh, rt.lib(), g.device
        if g.data_ptr() != sh.dxbuf.data_ptr():
            sh.dxbuf.copy_(g)
        ep = sh.next_epoch(K_OUT_DX)
        rt.check(lib.prb_ep_signal(sh.p_flags, sh.rank, sh.R, K_OUT_DX, ep, rt.stream_ptr(dev)), "prb_ep_signal")
        dx = torch.empty(route.T, sh.H, dtype=torch.bfloat16, device=dev)
        rt.check(lib.prb_ep_pull(sh.p_dx, route.idx.data_ptr(), route.pos.data_ptr(), None, None, dx.data_ptr(), None,
                                 sh.flags.data_ptr(), route.T, route.k, sh.H, sh.E, sh.R, K_OUT_DX, ep, _status(dev),
                                 rt.stream_ptr(dev)), "prb_ep_pull")
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, w, route: _Route):
        sh, lib, dev = route.sh, rt.lib(), yp.device
        if route.push_done is not None:          # the pull reads the positions the side-stream push wrote
            torch.cuda.current_stream(dev).wait_event(route.push_done)
        if yp.data_ptr() != sh.ybuf.data_ptr():
            sh.ybuf[:yp.shape[0]].copy_(yp)
        ep = sh.next_epoch(K_OUT_Y)
        route.ep_y = ep
        rt.check(lib.prb_ep_signal(sh.p_flags, sh.rank, sh.R, K_OUT_Y, ep, rt.stream_ptr(dev)), "prb_ep_signal")
        out = torch.empty(route.T, sh.H, dtype=torch.bfloat16, device=dev)
        wf = w.detach().float().contiguous()
        rt.check(lib.prb_ep_pull(sh.p_y, route.idx.data_ptr(), route.pos.data_ptr(), wf.data_ptr(), None,
                                 out.data_ptr(), None, sh.flags.data_ptr(), route.T, route.k, sh.H, sh.E, sh.R, K_OUT_Y,
                                 ep, _status(dev), rt.stream_ptr(dev)), "prb_ep_pull")
        ctx.route = route
        ctx.save_for_backward(wf)
        ctx.w_dtype = w.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        route = ctx.route
        (wf,) = ctx.saved_tensors
        sh, lib, dev = route.sh, rt.lib(), dout.device
        dout = dout.contiguous()
        # router-weight gradient: <y row, dout[t]> with the owners' y rows, which are still in place
        dw = torch.empty(route.T, route.k, dtype=torch.float32, device=dev)
        rt.check(lib.prb_ep_pull(sh.p_y, route.idx.data_ptr(), route.pos.data_ptr(), None, dout.data_ptr(), None,
                                 dw.data_ptr(), sh.flags.data_ptr(), route.T, route.k, sh.H, sh.E, sh.R, K_OUT_Y,
                                 route.ep_y, _status(dev), rt.stream_ptr(dev)), "prb_ep_pull")
        ep = sh.next_epoch(K_DATA_G)
        rt.check(lib.prb_ep_push(dout.data_ptr(), route.idx.data_ptr(), None, None, None, route.pos.data_ptr(),
                                 wf.data_ptr(), sh.p_g, sh.p_flags, None, sh.done.data_ptr(), route.T * route.k,
                                 route.k, sh.H, sh.E, sh.rank, sh.R, K_DATA_G, ep, sh.cap, _status(dev),
                                 rt.stream_ptr(dev)), "prb_ep_push")
        rt.check(lib.prb_ep_recv(sh.gbuf.data_ptr(), route.hist.data_ptr(), route.expert_offset.data_ptr(),
                                 sh.flags.data_ptr(), sh.rank, sh.R, sh.E, sh.H, K_DATA_G, ep, _status(dev),
                                 rt.stream_ptr(dev)), "prb_ep_recv")
        return sh.gbuf.view(sh.cap, sh.H), dw.to(ctx.w_dtype), None


class P2PDispatcher:
    """Drop-in for ``TorchA2ADispatcher``. ``capacity_factor`` bounds the rows one rank can
    receive as a multiple of the rows it sends (``T * k``); an overflow is reported through the
    kernel status word (``ops._runtime.check_status``)."""

    def __init__(self, group, ep: int, num_experts: int, capacity_factor: float | None = None,
                 max_tokens: int | None = None,
                 payload: str = "bf16", per_block: bool = False):
        if payload not in ("bf16", "fp8"):
            raise ValueError("payload must be 'bf16' or 'fp8'")
        self.payload = payload
        # per_block: the forward dispatch overlaps the first expert GEMM (rows pushed on a side stream, the GEMM's
        # loader waits per 128-row block); possible where the experts run their plain bf16 grouped GEMM
        self.per_block = per_block
        self.group, self.ep, self.E = group, ep, num_experts
        self.E_local = num_experts // ep
        # None: room for the worst case (all pairs of all ranks land on one rank), so a skewed router can never
        # overflow the buffers; a smaller factor trades that guarantee for memory
        self.capacity_factor = float(ep) if capacity_factor is None else capacity_factor
        # Tokens per rank and call the buffers are sized for. Every rank must derive the SAME
        # capacity: the symmetric buffers have one layout, and peers compute addresses inside each
        # other's allocation from it. When not given, the first call agrees on the maximum over the
        # ranks (one host synchronisation, once).
        self.max_tokens = max_tokens

    def _cap(self, k: int) -> int:
        T = self.max_tokens
        rows = int(T * k * self.capacity_factor) + self.E_local * 128
        return min(max(rows, 1024), self.ep * T * k + self.E_local * 128) // 128 * 128 + 128

    def __call__(self, experts, x, idx, w, counts):
        T, k = idx.shape
        dev = x.device
        lib = rt.lib()
        if self.max_tokens is None:
            t = torch.tensor([T], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            self.max_tokens = int(t.item())
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens in one call, but the dispatcher's buffers are sized for {self.max_tokens} "
                             "(pass max_tokens = tokens per rank and micro-batch)")
        sh = _Shared.get(self.group, self.ep, self.E, x.shape[1], self._cap(k), dev, self.payload == "fp8")
        idx = idx.contiguous()
        counts = counts.to(torch.int32).contiguous()
        local = moe_ops.build_plan(idx, counts, self.E)          # rank of every pair inside its expert
        route = _Route()
        route.sh, route.idx, route.slot, route.local_off, route.T, route.k = sh, idx, local.slot, local.expert_offset, T, k
        route.local, route.counts, route.push_done, route.block_rows = local, counts, None, None
        ep = sh.next_epoch(K_HIST)
        rt.check(lib.prb_ep_hist(counts.data_ptr(), sh.p_hist, sh.p_flags, sh.rank, sh.R, sh.E, K_HIST, ep,
                                 rt.stream_ptr(dev)), "prb_ep_hist")
        max_blocks = sh.cap // 128
        route.send_base = torch.empty(self.E, dtype=torch.int32, device=dev)
        route.expert_offset = torch.empty(self.E_local + 1, dtype=torch.int32, device=dev)
        route.block_expert = torch.empty(max_blocks, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        rt.check(lib.prb_ep_plan(sh.hist.data_ptr(), sh.flags.data_ptr(), sh.rank, sh.R, sh.E, K_HIST, ep, sh.cap,
                                 max_blocks, route.send_base.data_ptr(), route.expert_offset.data_ptr(),
                                 route.block_expert.data_ptr(), total.data_ptr(), _status(dev), rt.stream_ptr(dev)),
                 "prb_ep_plan")
        route.hist = sh.hist.clone()                              # the table is reused by the next call
        route.pos = torch.empty(T, k, dtype=torch.int32, device=dev)
        supports = getattr(experts, "supports_block_ready", None)
        per_block = (self.per_block and self.payload == "bf16" and supports is not None and supports(x)
                     and not stash.active())
        xin = _Dispatch.apply(x, route, per_block)
        # the experts write their output and their input gradient straight into the symmetric buffers
        xin._grad_out_buf = sh.dxbuf
        if per_block:
            yp = experts(xin, route.block_expert, route.expert_offset, out=sh.ybuf.view(sh.cap, sh.H),
                         block_ready=xin._blk_ready)
        else:
            try:
                yp = experts(xin, route.block_expert, route.expert_offset, out=sh.ybuf.view(sh.cap, sh.H))
            except TypeError:                       # an experts callable without the `out` argument
                yp = experts(xin, route.block_expert, route.expert_offset)
        return _Combine.apply(yp, w, route)
