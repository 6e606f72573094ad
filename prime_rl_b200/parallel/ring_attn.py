"""Ring form of context-parallel attention: K / V never exist as a whole on any rank.

Every rank keeps its own K / V chunks; in step s it holds the chunks of rank ``(r - s) mod cp``, computes the
partial attention of its local queries over them (output and log-sum-exp over that key range only) and merges it
into the running result::

    lse = logaddexp(lse_a, lse_b);  out = out_a exp(lse_a - lse) + out_b exp(lse_b - lse)

With the zig-zag token layout (rank r holds chunks r and 2 cp - 1 - r) every step is the same amount of work on
every rank: two chunk pairs per step (three in step 0, two of them diagonal). The backward pass walks the same
ring with the final output and log-sum-exp of the rows, so that every (row slice, key range) block yields exact
partial gradients: dQ is summed locally, the dK / dV partials go back to the rank that owns the keys.

Reference: src/prime_rl/trainer/models/layers/ring_attn.py:218-368 (ring of flash-attention calls with
log-sum-exp merging, backward ring that passes dK / dV along), src/prime_rl/utils/cp.py:73-95 (sharding).

Two exchanges:

``_RelayRing``   ``torch.distributed`` point-to-point: every rank passes the block it holds to the next rank while
                 it computes (works on gloo and NCCL); the dK / dV partials return through one all-to-all.
``_SymmRing``    one NVSwitch box: every rank publishes its K / V in symmetric memory once; the block of step
                 s + 1 is pulled straight from its owner (no relay: every peer is one hop away) into a local double
                 buffer by a copy kernel on a side stream while step s runs on the tensor cores. dK / dV partials
                 are written to a local slot per owner, and every owner sums its slot over all ranks with peer
                 loads in a fixed order (``slot_pull_reduce_kernel``).

The attention math of one block is ``csrc/flash_attn.cu: prb_flash_fwd_block`` / ``flash_attn_bwd.cu:
prb_flash_bwd_block`` (tcgen05; the query slice and the key range are given by their global offsets) on CUDA
and an fp32 PyTorch expression elsewhere.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

_KV_WRITTEN, _KV_READ, _DKV_WRITTEN, _DKV_READ = 0, 1, 2, 3


# ---------------------------------------------------------------------------------------------- block math
def _positions(cu, total, device):
    pos = torch.arange(total, device=device)
    doc = torch.searchsorted(cu[1:].to(torch.long).contiguous(), pos, right=True)
    return pos, doc


def block_fwd_ref(q, k, v, cu, total, q_off, k_off, window=None, scale=None):
    """fp32 partial attention of rows [q_off, q_off + Tq) over keys [k_off, k_off + Tk): (out, lse [Hq, Tq])."""
    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    pos, doc = _positions(cu, total, q.device)
    qp, kp = pos[q_off:q_off + Tq], pos[k_off:k_off + Tk]
    qd, kd = doc[q_off:q_off + Tq], doc[k_off:k_off + Tk]
    mask = (qd[:, None] == kd[None, :]) & (kp[None, :] <= qp[:, None])
    if window:
        mask &= qp[:, None] - kp[None, :] < window
    kf = k.float().repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("thd,shd->hts", q.float(), kf) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                  # -inf where no key is visible
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(mask[None], p, torch.zeros_like(p))
    return torch.einsum("hts,shd->thd", p, vf), lse, p


def _block_fwd(q, k, v, cu, total, q_off, k_off, window):
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
        from ..ops import flash_native

        return flash_native.flash_fwd_block(q.contiguous(), k, v, cu, total, q_off, k_off, window=window)
    out, lse, _ = block_fwd_ref(q, k, v, cu, total, q_off, k_off, window)
    return out, lse


def _block_bwd(dout, q, k, v, out, lse, cu, total, q_off, k_off, window):
    """Partial (dq, dk, dv) of one block given the rows' final ``out`` / ``lse``."""
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
        from ..ops import flash_native

        return flash_native.flash_bwd_block(dout, q.contiguous(), k, v, out.contiguous(), lse.contiguous(), cu, total,
                                            q_off, k_off, window=window)
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    pos, doc = _positions(cu, total, q.device)
    Tk = k.shape[0]
    qp, kp = pos[q_off:q_off + Tq], pos[k_off:k_off + Tk]
    mask = (doc[q_off:q_off + Tq, None] == doc[None, k_off:k_off + Tk]) & (kp[None, :] <= qp[:, None])
    if window:
        mask &= qp[:, None] - kp[None, :] < window
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q.float(), kf) * scale
    p = torch.where(mask[None], torch.exp(s - lse.float()[..., None]), torch.zeros_like(s))   # with the FINAL lse
    do = dout.float()
    delta = (do * out.float()).sum(-1).transpose(0, 1)               # [Hq, Tq]
    dp = torch.einsum("thd,shd->hts", do, vf)
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.einsum("hts,shd->thd", ds, kf)
    dk = torch.einsum("hts,thd->shd", ds, q.float()).view(Tk, Hkv, g, D).sum(2)
    dv = torch.einsum("hts,thd->shd", p, do).view(Tk, Hkv, g, D).sum(2)
    return dq, dk, dv


def merge_partial(acc, lse_acc, part, lse_part):
    """In-place merge of a partial result into (acc fp32 [T, H, D], lse_acc fp32 [H, T])."""
    if acc.is_cuda and part.dtype == torch.bfloat16 and acc.shape[-1] == 128:
        from ..ops import _runtime as rt

        T, H, _ = acc.shape
        rt.check(rt.lib().prb_attn_merge(acc.data_ptr(), lse_acc.data_ptr(), part.contiguous().data_ptr(),
                                         lse_part.contiguous().data_ptr(), T, H, rt.stream_ptr(acc.device)),
                 "prb_attn_merge")
        return
    lse_part = lse_part.float()
    new = torch.logaddexp(lse_acc, lse_part)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    wa = torch.exp(lse_acc - safe).transpose(0, 1)[..., None]        # -inf -> 0
    wp = torch.exp(lse_part - safe).transpose(0, 1)[..., None]
    acc.mul_(wa).add_(part.float() * wp)
    lse_acc.copy_(new)


# ---------------------------------------------------------------------------------------------- exchanges
class _RelayRing:
    """Blocks travel rank to rank with ``torch.distributed`` point-to-point calls, one hop per step, posted before
    the step's compute. dK / dV partials return with one all-to-all after the last step."""

    def __init__(self, cp):
        self.cp = cp

    def start(self, kv):
        self.cur, self.step, self.pending, self.nxt = kv, 0, None, None
        self._post()

    def _post(self):
        cp = self.cp
        if self.step + 1 >= cp.cp:
            return
        ranks = dist.get_process_group_ranks(cp.group)
        self.nxt = torch.empty_like(self.cur)
        ops = [dist.P2POp(dist.isend, self.cur, ranks[(cp.rank + 1) % cp.cp], group=cp.group),
               dist.P2POp(dist.irecv, self.nxt, ranks[(cp.rank - 1) % cp.cp], group=cp.group)]
        self.pending = dist.batch_isend_irecv(ops)

    def get(self, step):
        """K / V block of rank ``(rank - step) mod cp``; call with step = 0, 1, ... in order."""
        if step == 0:
            return self.cur
        for w in self.pending:
            w.wait()
        self.cur, self.step = self.nxt, step
        self._post()
        return self.cur

    def finish(self):
        pass

    def return_grads(self, parts):
        """parts[o]: this rank's dK / dV partial ([2, Tl, Hkv, D]) for owner o -> the sum over ranks of mine."""
        cp = self.cp
        send = torch.stack(parts).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=cp.group)
        return recv.float().sum(0)


class _SymmRing:
    """Symmetric-memory exchange for one NVSwitch box (see the module docstring)."""

    def __init__(self, cp, Tl, Hkv, D, device):
        from ..ops import _runtime as rt
        from .symm import SymmetricBuffer

        self.cp, self.rt, self.lib, self.device = cp, rt, rt.lib(), device
        R = cp.cp
        self.shape = (2, Tl, Hkv, D)
        self.n = 2 * Tl * Hkv * D
        self.blk_bytes = self.n * 2
        off_flags = (1 + R) * self.blk_bytes
        self.mem = SymmetricBuffer(cp.group, off_flags + 256, device, zero=True)
        self.own = self.mem.local(torch.bfloat16, 0, self.n).view(self.shape)
        self.slots = self.mem.local(torch.bfloat16, self.blk_bytes, R * self.n).view(R, *self.shape)
        self.flags = self.mem.local(torch.int32, off_flags, 4 * R)
        self.p_flags = self.mem.offset_ptrs(off_flags)
        self.slot_ptrs = self.mem.offset_ptrs(self.blk_bytes)
        self.recv = [torch.empty(self.shape, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.side = torch.cuda.Stream(device)
        self.epoch = 0
        self.free_ev = [None, None]          # main stream is done reading recv[i]
        self.ready_ev = [None, None]         # side stream has filled recv[i]

    def _barrier(self, kind):
        rt, cp = self.rt, self.cp
        stream = rt.stream_ptr(self.device)
        rt.check(self.lib.prb_ep_signal(self.p_flags, cp.rank, cp.cp, kind, self.epoch, stream), "prb_ep_signal")
        rt.check(self.lib.prb_ep_wait(self.flags.data_ptr(), cp.cp, kind, self.epoch,
                                      rt.status_tensor(self.device).data_ptr(), stream), "prb_ep_wait")

    def start(self, kv):
        self.epoch += 1
        self.own.copy_(kv)
        self._barrier(_KV_WRITTEN)           # every rank's block is in place before anybody pulls
        self.local = kv
        self.free_ev = [None, None]
        self._pull(1)

    def _pull(self, step):
        cp = self.cp
        if step >= cp.cp:
            return
        i = step & 1
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)                      # the pull starts once the barrier / the earlier steps are in the stream
        self.side.wait_event(ev)
        if self.free_ev[i] is not None:
            self.side.wait_event(self.free_ev[i])
        src = (cp.rank - step) % cp.cp
        with torch.cuda.stream(self.side):
            self.rt.check(self.lib.prb_peer_copy(self.mem.ptrs[src], self.recv[i].data_ptr(), self.blk_bytes, 32,
                                                 self.side.cuda_stream), "prb_peer_copy")
            self.ready_ev[i] = torch.cuda.Event()
            self.ready_ev[i].record(self.side)

    def get(self, step):
        if step == 0:
            return self.local
        i = step & 1
        main = torch.cuda.current_stream(self.device)
        main.wait_event(self.ready_ev[i])
        # the other buffer was read by step - 1, whose kernels are already in the main stream
        j = (step + 1) & 1
        self.free_ev[j] = torch.cuda.Event()
        self.free_ev[j].record(main)
        self._pull(step + 1)
        return self.recv[i]

    def finish(self):
        self._barrier(_KV_READ)              # nobody overwrites its block while a peer may still pull it

    def return_grads(self, parts):
        cp, rt = self.cp, self.rt
        for o, part in enumerate(parts):
            self.slots[o].copy_(part)
        self._barrier(_DKV_WRITTEN)
        out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.device)
        rt.check(self.lib.prb_slot_pull_reduce(self.slot_ptrs, cp.rank * self.blk_bytes, self.n, out.data_ptr(), cp.cp,
                                               rt.stream_ptr(self.device)), "prb_slot_pull_reduce")
        self._barrier(_DKV_READ)             # the slots are free again
        return out

    def close(self):
        self.mem.close()


# ---------------------------------------------------------------------------------------------- the ring
def _segments(cp, rank, Tl):
    """[(global offset, local row begin, local row end)] of the chunks rank ``rank`` holds."""
    if cp.layout == "zigzag":
        c = Tl // 2
        return [(rank * c, 0, c), ((2 * cp.cp - 1 - rank) * c, c, 2 * c)]
    return [(rank * Tl, 0, Tl)]


def _pairs(cp, src, Tl, window):
    """(q segment, k segment) pairs with at least one visible key when the local queries meet the keys of ``src``."""
    out = []
    for qo, qlo, qhi in _segments(cp, cp.rank, Tl):
        for ko, klo, khi in _segments(cp, src, Tl):
            if ko > qo:
                continue                                   # all keys after all queries
            if window and qo - (ko + (khi - klo) - 1) >= window:
                continue                                   # all keys outside the sliding window
            out.append(((qo, qlo, qhi), (ko, klo, khi)))
    return out


class RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cp, cu, total, window):
        Tl, Hq, D = q.shape
        ring = cp._ring(k)
        kv = torch.stack([k, v]).contiguous()
        acc = torch.zeros(Tl, Hq, D, dtype=torch.float32, device=q.device)
        lse = torch.full((Hq, Tl), float("-inf"), dtype=torch.float32, device=q.device)
        segs = _segments(cp, cp.rank, Tl)
        acc_s = [acc[lo:hi] for _, lo, hi in segs]
        lse_s = [torch.full((Hq, hi - lo), float("-inf"), dtype=torch.float32, device=q.device) for _, lo, hi in segs]
        ring.start(kv)
        for step in range(cp.cp):
            src = (cp.rank - step) % cp.cp
            blk = ring.get(step)
            for (qo, qlo, qhi), (ko, klo, khi) in _pairs(cp, src, Tl, window):
                part, lse_part = _block_fwd(q[qlo:qhi], blk[0, klo:khi], blk[1, klo:khi], cu, total, qo, ko, window)
                i = 0 if qlo == 0 else 1
                merge_partial(acc_s[i], lse_s[i], part, lse_part)
        ring.finish()
        for i, (_, lo, hi) in enumerate(segs):
            lse[:, lo:hi] = lse_s[i]
        out = acc.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.cfg = (cp, total, window)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        cp, total, window = ctx.cfg
        Tl = q.shape[0]
        ring = cp._ring(k)
        kv = torch.stack([k, v]).contiguous()
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        parts = [None] * cp.cp
        segs = _segments(cp, cp.rank, Tl)
        lse_s = [lse[:, lo:hi].contiguous() for _, lo, hi in segs]
        ring.start(kv)
        for step in range(cp.cp):
            src = (cp.rank - step) % cp.cp
            blk = ring.get(step)
            dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
            for (qo, qlo, qhi), (ko, klo, khi) in _pairs(cp, src, Tl, window):
                i = 0 if qlo == 0 else 1
                dq_p, dk_p, dv_p = _block_bwd(dout[qlo:qhi], q[qlo:qhi], blk[0, klo:khi], blk[1, klo:khi],
                                              out[qlo:qhi], lse_s[i], cu, total, qo, ko, window)
                dq[qlo:qhi] += dq_p
                dkv[0, klo:khi] += dk_p
                dkv[1, klo:khi] += dv_p
            parts[src] = dkv.to(k.dtype)
        ring.finish()
        dkv = ring.return_grads(parts)
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None
