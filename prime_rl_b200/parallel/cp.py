"""Context parallelism: the packed token stream is cut into chunks, every non-attention layer runs on the
local chunks, attention sees the whole (causal) context.

Token layout. ``contiguous``: rank r holds tokens ``[r T / cp, (r + 1) T / cp)``; with a causal mask rank r then
attends to r + 1 chunks of keys, so the last rank does ``2 cp / (cp + 1)`` times the average work and every
step waits for it. ``zigzag`` (default of the ``ring`` style): the stream is cut into ``2 cp`` chunks and rank
r holds chunks r and ``2 cp - 1 - r``; its two query slices together attend ``2 cp + 1`` chunk-units of keys
on every rank, so the attention kernels finish at the same time everywhere.

``ring``     (the reference's default, utils/cp.py:40-70 + layers/ring_attn.py:218-368): K/V of
             all chunks are all-gathered, local queries attend the keys up to the end of the
             local chunk, dK/dV are reduce-scattered in backward.
``ulysses``  (layers/ulysses_attn.py:53-152): all-to-all from sequence-sharded to head-sharded
             q/k/v, full-sequence attention on ``heads / cp`` heads, all-to-all back; KV heads are
             replicated when ``heads_kv < cp``.

Both run on ``torch.distributed`` collectives (NCCL / gloo) for the exchange and on the tcgen05
flash-attention kernels for the math (query-slice form for the all-gather path); per-token
outputs (logprobs, entropy) are gathered back along the sequence for the loss.

``ContextParallel(kv_exchange="ring" | "ring_p2p")`` replaces the all-gather of the ``ring`` style by a ring of K / V
blocks with one partial attention per step, merged through the log-sum-exp (``parallel/ring_attn.py``).

``ContextParallel(fused_kv_gather=True)`` moves the forward K / V exchange of the ``ring`` style into
the attention kernel: K and V live in a symmetric buffer, every rank writes its own chunk, and one
extra warp per CTA of the flash-attention forward pulls the chunks of the lower ranks over NVLink
with plain peer loads while the tensor cores already run (``csrc/flash_attn.cu:
flash_fwd_kernel<true>``); causality means a rank never needs the chunks above its own. The
backward uses the gathered copy and reduces dK / dV with the library collective as before.
"""

from __future__ import annotations

import math
from dataclasses import replace

import torch
import torch.distributed as dist

from ..models.layers import SeqInfo
from ..ops import attention as attn_ops


class _AllGatherSeq(torch.autograd.Function):
    """Concatenate the local chunks along dim 0. Backward: sum the incoming gradients over
    ranks and keep the local slice (reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, group, reduce_backward):
        ctx.group, ctx.reduce = group, reduce_backward
        n = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.rank, ctx.len = dist.get_rank(group), x.shape[0]
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, dy):
        if ctx.reduce:
            dy = dy.contiguous()
            dist.all_reduce(dy, group=ctx.group)
        return dy[ctx.rank * ctx.len:(ctx.rank + 1) * ctx.len].contiguous(), None, None


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all: input ``[cp, n, ...]`` (block i goes to rank i); backward is the
    same exchange."""

    @staticmethod
    def forward(ctx, x, group, p2p=None):
        ctx.group, ctx.p2p = group, p2p
        x = x.contiguous()
        if p2p is not None:
            return p2p(x)             # peer-memory exchange (parallel/p2p_a2a.py)
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()          # empty_like of a permuted gradient would keep its strides
        if ctx.p2p is not None:
            return ctx.p2p(dy), None, None
        dx = torch.empty_like(dy)
        dist.all_to_all_single(dx, dy, group=ctx.group)
        return dx, None, None


def attention_offset_ref(q, k, v, q_pos, k_pos, q_doc, k_doc, *, window=None, sinks=None, scale=None):
    """fp32 reference with explicit global positions / document ids for queries and keys."""
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kf = k.float().repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("thd,shd->hts", q.float(), kf) * scale
    mask = (q_doc[:, None] == k_doc[None, :]) & (k_pos[None, :] <= q_pos[:, None])
    if window is not None:
        mask &= q_pos[:, None] - k_pos[None, :] < window
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(Hq, 1, 1).expand(Hq, q.shape[0], 1)
        p = torch.softmax(torch.cat([s, sk], -1), -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    return torch.einsum("hts,shd->thd", p, vf).to(q.dtype)


_K_WRITTEN, _K_READ = 0, 1


class _FusedGatherAttention(torch.autograd.Function):
    """Forward: local chunk into the symmetric buffer, flag exchange, flash forward with the gather
    warp. Backward: the tcgen05 backward on the saved gathered K / V; dK / dV summed over ranks."""

    @staticmethod
    def forward(ctx, q, k, v, cp: "ContextParallel", cu, window):
        from ..ops import _runtime as rt
        from ..ops import flash_native

        Tl, Hkv, D = k.shape
        st = cp._kv_state(Tl, Hkv, D, q.device)
        lib, dev, R, rank = rt.lib(), q.device, cp.cp, cp.rank
        st["k"][rank * Tl:(rank + 1) * Tl].copy_(k)
        st["v"][rank * Tl:(rank + 1) * Tl].copy_(v)
        st["epoch"] += 1
        ep, stat, stream = st["epoch"], rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)
        rt.check(lib.prb_ep_signal(st["p_flags"], rank, R, _K_WRITTEN, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(st["flags"].data_ptr(), R, _K_WRITTEN, ep, stat, stream), "prb_ep_wait")
        out, lse = flash_native.flash_fwd_gather(q.contiguous(), st["k"], st["v"], st["mem"].c_ptrs, cu, rank, R,
                                                 st["counters"], window=window)
        # every rank is done reading my chunk before the next layer overwrites it
        rt.check(lib.prb_ep_signal(st["p_flags"], rank, R, _K_READ, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(st["flags"].data_ptr(), R, _K_READ, ep, stat, stream), "prb_ep_wait")
        hi = (rank + 1) * Tl
        kg, vg = torch.zeros_like(st["k"]), torch.zeros_like(st["v"])      # keys above the local chunk are never read
        kg[:hi].copy_(st["k"][:hi])
        vg[:hi].copy_(st["v"][:hi])
        ctx.save_for_backward(q, kg, vg, out, lse, cu)
        ctx.cfg = (cp, window, Tl)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import flash_native

        q, kg, vg, out, lse, cu = ctx.saved_tensors
        cp, window, Tl = ctx.cfg
        dq, dk, dv = flash_native.flash_bwd(dout, q, kg, vg, out, lse, cu, window=window, q_offset=cp.rank * Tl)
        dist.all_reduce(dk, group=cp.group)
        dist.all_reduce(dv, group=cp.group)
        lo = cp.rank * Tl
        return dq, dk[lo:lo + Tl].contiguous(), dv[lo:lo + Tl].contiguous(), None, None, None


class ContextParallel:
    def __init__(self, group, cp: int, rank: int, style: str = "ring", p2p_all_to_all: bool = False,
                 fused_kv_gather: bool = False, layout: str | None = None, kv_exchange: str = "nccl"):
        self.group, self.cp, self.rank, self.style = group, cp, rank, style
        self.fused_kv_gather, self._kv = fused_kv_gather, None
        # "ring" / "ring_p2p": step-by-step K / V blocks with log-sum-exp merging (parallel/ring_attn.py)
        self.kv_exchange, self._ring_state = kv_exchange, None
        # the in-kernel K / V gather and the Ulysses exchange address contiguous chunks
        self.layout = layout or ("zigzag" if style == "ring" and not fused_kv_gather else "contiguous")
        if self.layout == "zigzag" and (style != "ring" or fused_kv_gather):
            raise ValueError("the zigzag token layout goes with cp_style = 'ring' and the all-gather K / V exchange")
        # Ulysses exchanges over NVLink peer memory instead of NCCL (built on first use, sized by the first block)
        self.use_p2p, self._p2p = p2p_all_to_all, None

    def _kv_state(self, Tl: int, Hkv: int, D: int, device) -> dict:
        """Symmetric K / V buffer of the fused-gather path: [K: T rows | V: T rows | counters | flags]."""
        key = (Tl, Hkv, D)
        if self._kv is None or self._kv["key"] != key:
            from .symm import SymmetricBuffer

            if self._kv is not None:
                self._kv["mem"].close()
            T = Tl * self.cp
            half = T * Hkv * D * 2
            off_cnt = 2 * half
            off_flags = off_cnt + 256
            mem = SymmetricBuffer(self.group, off_flags + 256, device, zero=True)
            self._kv = {"key": key, "mem": mem, "epoch": 0,
                        "k": mem.local(torch.bfloat16, 0, T * Hkv * D).view(T, Hkv, D),
                        "v": mem.local(torch.bfloat16, half, T * Hkv * D).view(T, Hkv, D),
                        "counters": mem.local(torch.int32, off_cnt, self.cp + 1),
                        "flags": mem.local(torch.int32, off_flags, 2 * self.cp),
                        "p_flags": mem.offset_ptrs(off_flags)}
        return self._kv

    def _exchange(self, x):
        if self.use_p2p and x.is_cuda:
            if self._p2p is None:
                from .p2p_a2a import P2PAllToAll

                self._p2p = P2PAllToAll(self.group, 4 * x[0].numel() * x.element_size(), x.device)
            return _AllToAll.apply(x, self.group, self._p2p)
        return _AllToAll.apply(x, self.group)

    # ------------------------------------------------------------------ sharding
    def shard(self, t: torch.Tensor) -> torch.Tensor:
        if self.layout == "zigzag":
            c = t.shape[0] // (2 * self.cp)
            a, b = self.rank, 2 * self.cp - 1 - self.rank
            return torch.cat([t[a * c:(a + 1) * c], t[b * c:(b + 1) * c]], 0)
        n = t.shape[0] // self.cp
        return t[self.rank * n:(self.rank + 1) * n]

    def _to_global_order(self, gathered: torch.Tensor) -> torch.Tensor:
        """Rank-major concatenation of the local rows (what an all-gather returns) -> global token order."""
        if self.layout != "zigzag":
            return gathered
        cp = self.cp
        c = gathered.shape[0] // (2 * cp)
        v = gathered.view(cp, 2, c, *gathered.shape[1:])
        # global chunk j sits on rank j (first half) for j < cp, on rank 2 cp - 1 - j (second half) otherwise
        ranks = torch.tensor([j if j < cp else 2 * cp - 1 - j for j in range(2 * cp)], device=gathered.device)
        halves = torch.tensor([0 if j < cp else 1 for j in range(2 * cp)], device=gathered.device)
        return v[ranks, halves].reshape(gathered.shape)

    def shard_inputs(self, ids, labels, inv_temp, seq: SeqInfo):
        T = ids.shape[0]
        unit = 2 * self.cp if self.layout == "zigzag" else self.cp
        if T % unit:
            raise ValueError(f"packed length {T} is not a multiple of {unit} (cp = {self.cp}, {self.layout} layout; "
                             "set pad_to_multiple_of)")
        local = replace(seq, position_ids=self.shard(seq.position_ids), cp=self)
        if seq.routed_experts is not None:
            local.routed_experts = self.shard(seq.routed_experts)
        local.full_cu_seqlens = seq.cu_seqlens
        local.full_len = T
        return self.shard(ids), self.shard(labels), self.shard(inv_temp), local

    def gather_outputs(self, logprobs, entropy):
        lp = self._to_global_order(_AllGatherSeq.apply(logprobs, self.group, False))
        with torch.no_grad():
            ent = self._to_global_order(_AllGatherSeq.apply(entropy, self.group, False))
        return lp, ent

    # ------------------------------------------------------------------ recurrent mixers
    # A recurrent state cannot be cut along the sequence, so the state-carrying mixers (Mamba-2, gated delta-net) trade
    # the sequence split for a head split: every rank gets the WHOLE sequence of its own heads, runs convolution and
    # scan on them, and goes back (reference: src/prime_rl/trainer/models/nemotron_h/mamba.py:20-48). Contiguous
    # token layout only (``cp_style = "ulysses"``).
    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """``[Tl, F]`` (all features of the local tokens) -> ``[T, F / cp]`` (this rank's feature block of all tokens)."""
        if self.layout != "contiguous":
            raise ValueError("recurrent mixers under context parallelism need the contiguous token layout "
                             "(cp_style = 'ulysses')")
        Tl, F = x.shape
        x = x.reshape(Tl, self.cp, F // self.cp).permute(1, 0, 2).contiguous()
        return self._exchange(x).reshape(self.cp * Tl, F // self.cp)

    def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """``[T, F / cp]`` -> ``[Tl, F]``: inverse of ``seq_to_heads``."""
        T, Fl = x.shape
        x = self._exchange(x.reshape(self.cp, T // self.cp, Fl).contiguous())          # [cp (feature block), Tl, Fl]
        return x.permute(1, 0, 2).reshape(T // self.cp, self.cp * Fl)

    def gather_seq(self, x: torch.Tensor) -> torch.Tensor:
        """``[Tl, F]`` -> ``[T, F]`` on every rank (features every rank needs whole: the B / C groups of Mamba-2);
        gradients are summed over the ranks."""
        return _AllGatherSeq.apply(x.contiguous(), self.group, True)

    def global_rows(self, Tl: int, device) -> torch.Tensor:
        """Global token index of every local row."""
        if self.layout == "zigzag":
            c = Tl // 2
            a, b = self.rank, 2 * self.cp - 1 - self.rank
            return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])
        return torch.arange(self.rank * Tl, (self.rank + 1) * Tl, device=device)

    def gather_rows(self, x: torch.Tensor, grad: bool = True) -> torch.Tensor:
        """``[Tl, ...]`` -> ``[T, ...]`` in global token order on every rank (small per-token features that every query
        may read: latent K / V rows, indexer keys); with ``grad`` the gradients are summed over the ranks."""
        if grad:
            return self._to_global_order(_AllGatherSeq.apply(x.contiguous(), self.group, True))
        with torch.no_grad():
            return self._to_global_order(_AllGatherSeq.apply(x.contiguous(), self.group, False))

    def full_positions(self, seq: SeqInfo) -> torch.Tensor:
        """Position of every token of the whole packed sequence inside its document."""
        cu = seq.full_cu_seqlens.to(torch.long)
        pos = torch.arange(seq.full_len, device=cu.device)
        doc = torch.searchsorted(cu[1:].contiguous(), pos, right=True)
        return (pos - cu[doc]).to(torch.int32)

    # ------------------------------------------------------------------ attention
    def _doc_ids(self, cu, T, device):
        pos = torch.arange(T, device=device)
        return torch.searchsorted(cu[1:].to(torch.long).contiguous(), pos, right=True)

    def attention(self, q, k, v, seq: SeqInfo, *, window=None, sinks=None, backend="auto"):
        if self.style == "ulysses":
            return self._ulysses(q, k, v, seq, window, sinks, backend)
        return self._gather_kv(q, k, v, seq, window, sinks, backend)

    def _ring(self, k):
        """Exchange object of the ring form for K / V chunks shaped like ``k``."""
        from .ring_attn import _RelayRing, _SymmRing

        if self.kv_exchange == "ring_p2p" and k.is_cuda and k.dtype == torch.bfloat16:
            key = tuple(k.shape)
            if self._ring_state is None or self._ring_state[0] != key:
                if self._ring_state is not None:
                    self._ring_state[1].close()
                self._ring_state = (key, _SymmRing(self, *key, k.device))
            return self._ring_state[1]
        return _RelayRing(self)

    def _gather_kv(self, q, k, v, seq, window, sinks, backend):
        Tl, T = q.shape[0], seq.full_len
        if self.kv_exchange in ("ring", "ring_p2p") and sinks is None:
            from .ring_attn import RingAttention

            cu = seq.full_cu_seqlens.to(torch.int32) if q.is_cuda else seq.full_cu_seqlens
            return RingAttention.apply(q, k.contiguous(), v.contiguous(), self, cu, T, window)
        if (self.fused_kv_gather and q.is_cuda and sinks is None and q.dtype == torch.bfloat16 and q.shape[-1] == 128
                and self.cp <= 8):
            return _FusedGatherAttention.apply(q, k.contiguous(), v.contiguous(), self,
                                               seq.full_cu_seqlens.to(torch.int32), window)
        kg = self._to_global_order(_AllGatherSeq.apply(k, self.group, True))
        vg = self._to_global_order(_AllGatherSeq.apply(v.contiguous(), self.group, True))
        cu = seq.full_cu_seqlens
        if self.layout == "zigzag":
            # two query slices per rank: chunk r against keys [0, (r + 1) c) and chunk 2 cp - 1 - r against keys
            # [0, (2 cp - r) c): 2 cp + 1 chunk-units of keys on every rank
            c = Tl // 2
            outs = []
            for half, chunk in ((0, self.rank), (1, 2 * self.cp - 1 - self.rank)):
                qs, lo = q[half * c:(half + 1) * c], chunk * c
                if q.is_cuda and sinks is None and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
                    max_len = int((cu[1:] - cu[:-1]).max())
                    outs.append(attn_ops.attention(qs.contiguous(), kg, vg, cu.to(torch.int32), max_len, causal=True,
                                                   window=window, backend="tcgen05", q_offset=lo))
                else:
                    doc = self._doc_ids(cu, T, q.device)
                    pos = torch.arange(T, device=q.device)
                    hi = lo + c
                    outs.append(attention_offset_ref(qs, kg[:hi], vg[:hi], pos[lo:hi], pos[:hi], doc[lo:hi], doc[:hi],
                                                     window=window, sinks=sinks))
            return torch.cat(outs, 0)
        lo, hi = self.rank * Tl, (self.rank + 1) * Tl
        if q.is_cuda and sinks is None and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
            # the tcgen05 kernels take a query slice directly: local rows [lo, hi) of the global
            # sequence against all gathered keys (causality hides the keys past hi); the
            # backward returns this rank's dK / dV for every key, which _AllGatherSeq reduces
            max_len = int((cu[1:] - cu[:-1]).max())
            return attn_ops.attention(q.contiguous(), kg, vg, cu.to(torch.int32), max_len, causal=True, window=window,
                                      backend="tcgen05", q_offset=lo)
        doc = self._doc_ids(cu, T, q.device)
        pos = torch.arange(T, device=q.device)
        return attention_offset_ref(q, kg[:hi], vg[:hi], pos[lo:hi], pos[:hi], doc[lo:hi], doc[:hi], window=window,
                                    sinks=sinks)

    def _ulysses(self, q, k, v, seq, window, sinks, backend):
        cp, Tl = self.cp, q.shape[0]
        Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
        if Hq % cp:
            raise ValueError(f"ulysses needs num_attention_heads ({Hq}) divisible by cp ({cp})")
        if Hkv < cp:
            if cp % Hkv:
                raise ValueError("ulysses needs cp | heads_kv or heads_kv | cp")
            k = k.repeat_interleave(cp // Hkv, dim=1)
            v = v.repeat_interleave(cp // Hkv, dim=1)
            Hkv = cp
        elif Hkv % cp:
            raise ValueError("ulysses needs cp | heads_kv or heads_kv | cp")

        def seq_to_head(x, H):      # [Tl, H, D] -> [T, H/cp, D]
            x = x.reshape(Tl, cp, H // cp, D).permute(1, 0, 2, 3).contiguous()      # [cp, Tl, H/cp, D]
            return self._exchange(x).reshape(cp * Tl, H // cp, D)

        def head_to_seq(x, H):      # [T, H/cp, D] -> [Tl, H, D]
            x = self._exchange(x.reshape(cp, Tl, H // cp, D).contiguous())   # [cp(head blk), Tl, H/cp, D]
            return x.permute(1, 0, 2, 3).reshape(Tl, H, D)

        qf, kf, vf = seq_to_head(q, Hq), seq_to_head(k, Hkv), seq_to_head(v.contiguous(), Hkv)
        local_sinks = None
        if sinks is not None:
            h0 = self.rank * (Hq // cp)
            local_sinks = sinks[h0:h0 + Hq // cp]
        cu = seq.full_cu_seqlens
        max_len = int((cu[1:] - cu[:-1]).max())
        o = attn_ops.attention(qf, kf, vf, cu, max_len, causal=True, window=window, sinks=local_sinks, backend=backend)
        return head_to_seq(o, Hq)
