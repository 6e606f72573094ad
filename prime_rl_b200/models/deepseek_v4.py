"""DeepSeek-V4 building blocks on packed ``[T, ...]`` activations.

What sets the family apart from the flag-driven decoder in ``layers.py``:

* the residual is ``hc_mult`` parallel streams ``[T, hc, hidden]`` tied together by
  manifold-constrained hyper-connections: per sublayer one projection of the normalised streams
  gives "pre" weights (collapse the streams into the sublayer input), "post" weights (spread the
  sublayer output back) and an ``hc x hc`` mixing matrix pushed towards doubly-stochastic by
  Sinkhorn iterations; a "hyper head" collapses the streams before the final norm;
* attention is shared-KV multi-query (one ``head_dim`` vector per token is key and value of every
  head) over explicit slots: a causal sliding window of recent tokens, plus, on compressed layers,
  entries that pool ``compress_rate`` consecutive tokens each (softmax-gated pooling, RMSNorm,
  rotary at the entry's first position). "Compressed sparse" layers pool 2 overlapping series at a
  fine rate and let a lightning indexer pick ``index_topk`` entries per query; "heavily
  compressed" layers pool at a coarse rate and read every completed entry. Per-head attention
  sinks; the output is de-rotated (values carry the keys' rotation) and leaves through a grouped
  low-rank projection;
* MoE layers score with ``sqrt(softplus(.))``; the first ``num_hash_layers`` route by a frozen
  token-id table, the rest by top-k with a selection bias; experts use a clamped SwiGLU.

Parameter names follow the reference modules (src/prime_rl/trainer/models/deepseek_v4/
hyperconnections.py:19-97, attention.py:408-777, moe.py:35-259, modeling_deepseek_v4.py:40-75).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import moe as moe_ops
from ..ops import sparse_mla
from .config import ModelArch
from .layers import DenseMLP, Linear, MoE, RMSNorm, SeqInfo

IGNORE_SLOT = -1


def unweighted_rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps).to(x.dtype)


def rope_interleaved(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, conj: bool = False) -> torch.Tensor:
    """Rotates the trailing ``2 * len(inv_freq)`` channels of ``x [T, heads, D]`` (pairs stored
    adjacently: ``(x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin)``) by ``pos [T]``; ``conj`` rotates
    by the opposite angle."""
    rd = inv_freq.numel() * 2
    ang = pos.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if conj:
        sin = -sin
    nope, rope = x[..., :-rd], x[..., -rd:].float()
    x0, x1 = rope[..., 0::2], rope[..., 1::2]
    rot = torch.stack((x0 * cos - x1 * sin, x1 * cos + x0 * sin), dim=-1).flatten(-2)
    return torch.cat([nope, rot.to(x.dtype)], dim=-1)


# ---------------------------------------------------------------------- hyper-connections
class HyperConnection(nn.Module):
    def __init__(self, arch: ModelArch, dtype=None, device=None):
        super().__init__()
        hc = arch.hc_mult
        self.hc, self.iters, self.eps, self.norm_eps = hc, arch.hc_sinkhorn_iters, arch.hc_eps, arch.rms_norm_eps
        mix = (2 + hc) * hc
        self.fn = nn.Parameter(torch.empty(mix, hc * arch.hidden_size, dtype=torch.float32, device=device))
        self.base = nn.Parameter(torch.zeros(mix, dtype=torch.float32, device=device))
        self.scale = nn.Parameter(torch.ones(3, dtype=torch.float32, device=device))

    def forward(self, streams: torch.Tensor):
        """``streams [T, hc, H]`` -> ``post [T, hc]``, ``comb [T, hc, hc]``, ``collapsed [T, H]``."""
        hc = self.hc
        flat = unweighted_rms_norm(streams.flatten(1).float(), self.norm_eps)
        pre_w, post_w, comb_w = F.linear(flat, self.fn).split([hc, hc, hc * hc], dim=-1)
        pre_b, post_b, comb_b = self.base.split([hc, hc, hc * hc])
        pre = torch.sigmoid(pre_w * self.scale[0] + pre_b) + self.eps
        post = 2 * torch.sigmoid(post_w * self.scale[1] + post_b)
        comb = torch.softmax(comb_w.view(-1, hc, hc) * self.scale[2] + comb_b.view(hc, hc), dim=-1) + self.eps
        comb = comb / (comb.sum(-2, keepdim=True) + self.eps)
        for _ in range(self.iters - 1):
            comb = comb / (comb.sum(-1, keepdim=True) + self.eps)
            comb = comb / (comb.sum(-2, keepdim=True) + self.eps)
        collapsed = (pre.unsqueeze(-1) * streams).sum(1).to(streams.dtype)
        return post, comb, collapsed

    @staticmethod
    def merge(streams: torch.Tensor, out: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
        dt = streams.dtype
        return post.to(dt).unsqueeze(-1) * out.unsqueeze(1) + torch.matmul(comb.to(dt).transpose(-1, -2), streams)


class HyperHead(nn.Module):
    def __init__(self, arch: ModelArch, dtype=None, device=None):
        super().__init__()
        hc = arch.hc_mult
        self.eps, self.norm_eps = arch.hc_eps, arch.rms_norm_eps
        self.hc_fn = nn.Parameter(torch.empty(hc, hc * arch.hidden_size, dtype=torch.float32, device=device))
        self.hc_base = nn.Parameter(torch.zeros(hc, dtype=torch.float32, device=device))
        self.hc_scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device))

    def forward(self, streams: torch.Tensor) -> torch.Tensor:
        flat = unweighted_rms_norm(streams.flatten(1).float(), self.norm_eps)
        pre = torch.sigmoid(F.linear(flat, self.hc_fn) * self.hc_scale + self.hc_base) + self.eps
        return (pre.unsqueeze(-1) * streams).sum(1).to(streams.dtype)


# ---------------------------------------------------------------------- packing bookkeeping
class CompressionLayout:
    """Entries of one compress rate: document ``d`` of length ``L`` owns ``L // rate`` entries, entry
    ``e`` pools tokens ``[start_d + e * rate, start_d + (e + 1) * rate)``; trailing tokens own none."""

    def __init__(self, cu_seqlens: torch.Tensor, rate: int):
        dev = cu_seqlens.device
        starts = cu_seqlens[:-1].long()
        counts = (cu_seqlens[1:].long() - starts) // rate
        self.entry_doc = torch.repeat_interleave(torch.arange(counts.numel(), device=dev), counts)
        self.first_entry_of_doc = counts.cumsum(0) - counts
        n = int(counts.sum())
        self.entry_local = torch.arange(n, device=dev) - self.first_entry_of_doc[self.entry_doc]
        self.entry_tok = (starts[self.entry_doc, None] + (self.entry_local * rate)[:, None]
                          + torch.arange(rate, device=dev)[None, :])
        self.max_per_doc = int(counts.max()) if counts.numel() else 0
        self.rate, self.n = rate, n


def packed_context(seq: SeqInfo, arch: ModelArch) -> dict:
    """Built once per forward and kept on ``seq.shared``: document id of every token, the sliding
    window's slot indices, and one ``CompressionLayout`` per compress rate. Under context parallelism the
    tokens are the local ones, their slot indices and the layouts are those of the whole sequence, and ``gather``
    maps per-token rows of the local tokens to the rows of all tokens (``parallel/cp.py: gather_rows``)."""
    if seq.shared is None:
        seq.shared = {}
    ctx = seq.shared.get("dsv4")
    if ctx is None and seq.cp is not None:
        cp, pos = seq.cp, seq.position_ids.long()
        me = cp.global_rows(pos.shape[0], pos.device)
        cu = seq.full_cu_seqlens.to(pos.device)
        doc = torch.searchsorted(cu[1:].long().contiguous(), me, right=True)
        back = torch.arange(arch.sliding_window, device=pos.device)
        win = me[:, None] - back[None, :]
        win = torch.where(back[None, :] <= pos[:, None], win, torch.full_like(win, IGNORE_SLOT))
        rates = sorted({r for r in (arch.csa_compress_rate, arch.hca_compress_rate) if r})
        ctx = {"doc": doc, "window": win, "layouts": {r: CompressionLayout(cu, r) for r in rates},
               "gather": cp.gather_rows, "gather_nograd": lambda t: cp.gather_rows(t, grad=False),
               "total": int(seq.full_len)}
        seq.shared["dsv4"] = ctx
    if ctx is None:
        pos = seq.position_ids.long()
        T = pos.shape[0]
        me = torch.arange(T, device=pos.device)
        doc = torch.cumsum((pos == 0).long(), 0) - 1
        back = torch.arange(arch.sliding_window, device=pos.device)
        win = me[:, None] - back[None, :]                              # most recent token first
        win = torch.where(back[None, :] <= pos[:, None], win, torch.full_like(win, IGNORE_SLOT))
        rates = sorted({r for r in (arch.csa_compress_rate, arch.hca_compress_rate) if r})
        ctx = {"doc": doc, "window": win, "layouts": {r: CompressionLayout(seq.cu_seqlens, r) for r in rates}}
        seq.shared["dsv4"] = ctx
    return ctx


# ---------------------------------------------------------------------- compressors
class Compressor(nn.Module):
    """``C[e, d] = sum_s softmax_s(gate[e, s, d] + position_bias[s, d]) * kv[e, s, d]`` over the tokens
    ``s`` of entry ``e``; with ``n_series == 2`` entry ``e`` also pools a second series from entry
    ``e - 1``'s tokens (overlapping windows; a document's first entry has no predecessor)."""

    def __init__(self, arch: ModelArch, head_dim: int, rate: int, n_series: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.head_dim, self.rate, self.n_series = arch, head_dim, rate, n_series
        std = arch.initializer_range
        self.kv_proj = Linear(arch.hidden_size, n_series * head_dim, std=std, dtype=dtype, device=device)
        self.gate_proj = Linear(arch.hidden_size, n_series * head_dim, std=std, dtype=dtype, device=device)
        self.position_bias = nn.Parameter(torch.zeros(rate, n_series * head_dim, dtype=torch.float32, device=device))
        self.kv_norm = RMSNorm(head_dim, arch.rms_norm_eps, dtype=dtype, device=device)
        from ..ops import inv_freq

        self.register_buffer("inv_freq", inv_freq(arch.qk_rope_head_dim, arch.compress_rope_theta, device=device),
                             persistent=False)

    def compress(self, x: torch.Tensor, layout: CompressionLayout, gather=None) -> torch.Tensor:
        """``x [T, hidden]`` -> entries ``[n_entries, head_dim]`` (rotated at their first position). ``gather``
        (context parallelism): maps the local tokens' projections to those of the whole sequence, which ``layout``
        then describes; every rank forms all entries."""
        D = self.head_dim
        kvp, gp = self.kv_proj(x), self.gate_proj(x)
        if gather is not None:
            kvp, gp = gather(kvp), gather(gp)
        kv = kvp[layout.entry_tok]                                      # [n, rate, series * D]
        gate = gp[layout.entry_tok].float() + self.position_bias
        if self.n_series == 2:
            prev = (torch.arange(layout.n, device=x.device) - 1).clamp(min=0)
            first = (layout.entry_local == 0)[:, None, None]
            kv = torch.cat([kv[prev, :, :D].masked_fill(first, 0.0), kv[..., D:]], dim=1)
            gate = torch.cat([gate[prev, :, :D].masked_fill(first, float("-inf")), gate[..., D:]], dim=1)
        w = gate.softmax(dim=1).to(kv.dtype)
        c = self.kv_norm((kv * w).sum(1))
        return rope_interleaved(c.unsqueeze(1), layout.entry_local * self.rate, self.inv_freq).squeeze(1)

    def pool(self, kvp: torch.Tensor, gp: torch.Tensor, first_entry: int, has_prev: bool) -> torch.Tensor:
        """Entries from the projections of their source tokens (rollout engine: entries are formed as their tokens
        arrive). ``kvp`` / ``gp``: ``kv_proj(x)`` / ``gate_proj(x)`` of the consecutive tokens of entries
        ``first_entry - 1`` (only when ``has_prev``: the second series pools from it) ``, first_entry, ...``; returns
        the entries from ``first_entry`` on, rotated at their first position."""
        D, R = self.head_dim, self.rate
        n_all = kvp.shape[0] // R
        kv = kvp.view(n_all, R, -1)
        gate = gp.float().view(n_all, R, -1) + self.position_bias
        if self.n_series == 2:
            cur_kv, cur_g = kv[1:] if has_prev else kv, gate[1:] if has_prev else gate
            if has_prev:
                prev_kv, prev_g = kv[:-1, :, :D], gate[:-1, :, :D]
            else:                   # the sequence's first entry has no predecessor; later ones of this call do
                prev_kv = torch.cat([torch.zeros_like(kv[:1, :, :D]), kv[:-1, :, :D]], 0)
                prev_g = torch.cat([torch.full_like(gate[:1, :, :D], float("-inf")), gate[:-1, :, :D]], 0)
            kv = torch.cat([prev_kv, cur_kv[..., D:]], dim=1)
            gate = torch.cat([prev_g, cur_g[..., D:]], dim=1)
        elif has_prev:
            kv, gate = kv[1:], gate[1:]
        n = kv.shape[0]
        w = gate.softmax(dim=1).to(kv.dtype)
        c = self.kv_norm((kv * w).sum(1))
        first = torch.arange(first_entry, first_entry + n, device=kvp.device) * R
        return rope_interleaved(c.unsqueeze(1), first, self.inv_freq).squeeze(1)

    def engine_entries(self, eng, store: dict, key, x: torch.Tensor, L: int) -> torch.Tensor:
        """All completed entries of one sequence after its ``x.shape[0]`` new tokens (``L`` tokens before them). The
        sequence keeps the entries made so far and the projections of the tokens that later entries still need."""
        R = self.rate
        st = store.setdefault(key, {"n": 0, "tail_start": 0, "kvp": None, "gp": None})
        if L == 0:
            st.update(n=0, tail_start=0, kvp=None, gp=None)
        kvp, gp = self.kv_proj(x), self.gate_proj(x)
        if st["kvp"] is not None:
            kvp, gp = torch.cat([st["kvp"], kvp], 0), torch.cat([st["gp"], gp], 0)
        total = (L + x.shape[0]) // R
        done = st["n"]
        entries = eng.append(store, (key, "entries"), x.new_zeros(0, self.head_dim), done)
        if total > done:
            has_prev = self.n_series == 2 and done > 0
            lo = (done - 1 if has_prev else done) * R - st["tail_start"]
            hi = total * R - st["tail_start"]
            new = self.pool(kvp[lo:hi], gp[lo:hi], done, has_prev)
            entries = eng.append(store, (key, "entries"), new.to(x.dtype), done)
            st["n"] = total
        keep_from = (max(total - 1, 0) if self.n_series == 2 else total) * R        # tokens later entries still read
        cut = keep_from - st["tail_start"]
        st["kvp"], st["gp"], st["tail_start"] = kvp[cut:], gp[cut:], keep_from
        return entries

    def readable_entries(self, position_ids: torch.Tensor) -> torch.Tensor:
        """How many entries of its own document query ``t`` may read: an entry becomes readable once
        the query has reached its last source token."""
        return (position_ids.long() + 1) // self.rate


class LightningIndexer(nn.Module):
    def __init__(self, arch: ModelArch, dtype=None, device=None):
        super().__init__()
        self.arch, self.nh, self.hd = arch, arch.index_n_heads, arch.index_head_dim
        std = arch.initializer_range
        self.compressor = Compressor(arch, self.hd, arch.csa_compress_rate, 2, dtype=dtype, device=device)
        self.q_b_proj = Linear(arch.q_lora_rank, self.nh * self.hd, std=std, dtype=dtype, device=device)
        self.weights_proj = Linear(arch.hidden_size, self.nh, std=std, dtype=dtype, device=device)
        for p in self.parameters():          # returns integer indices: nothing to differentiate
            p.requires_grad_(False)

    @torch.no_grad()
    def forward(self, x, q_residual, seq: SeqInfo, ctx: dict) -> torch.Tensor:
        layout = ctx["layouts"][self.compressor.rate]
        entries = self.compressor.compress(x, layout, ctx.get("gather_nograd"))
        T = x.shape[0]
        q = rope_interleaved(self.q_b_proj(q_residual).view(T, self.nh, self.hd), seq.position_ids,
                             self.compressor.inv_freq)
        start = layout.first_entry_of_doc[ctx["doc"]].int()
        stop = (start + self.compressor.readable_entries(seq.position_ids)).int()
        if layout.n == 0:
            return torch.full((T, self.arch.index_topk), IGNORE_SLOT, dtype=torch.long, device=x.device)
        picks = sparse_mla.dsa_indexer_topk(q, entries, self.weights_proj(x), start, stop, self.arch.index_topk).long()
        return torch.where(picks < layout.n, picks, torch.full_like(picks, IGNORE_SLOT))

    @torch.no_grad()
    def engine_picks(self, eng, store: dict, layer: int, x, q_residual, pos: torch.Tensor, L: int) -> torch.Tensor:
        """Rollout engine: the selection for the new tokens of one sequence over its own indexer entries."""
        entries = self.compressor.engine_entries(eng, store, (layer, "idx"), x, L)
        n = x.shape[0]
        if entries.shape[0] == 0:
            return torch.full((n, self.arch.index_topk), IGNORE_SLOT, dtype=torch.long, device=x.device)
        q = rope_interleaved(self.q_b_proj(q_residual).view(n, self.nh, self.hd), pos, self.compressor.inv_freq)
        stop = self.compressor.readable_entries(pos).int()
        picks = sparse_mla.dsa_indexer_topk(q, entries, self.weights_proj(x), torch.zeros_like(stop), stop,
                                            self.arch.index_topk).long()
        return torch.where(picks < entries.shape[0], picks, torch.full_like(picks, IGNORE_SLOT))


class GroupedLinear(nn.Module):
    """Block-diagonal projection: group ``g`` of the input maps to its own ``out / groups`` channels."""

    def __init__(self, in_per_group: int, out_features: int, groups: int, std: float, dtype=None, device=None):
        super().__init__()
        self.groups = groups
        self.weight = nn.Parameter(torch.empty(out_features, in_per_group, dtype=dtype, device=device))
        self.std = std

    def forward(self, x: torch.Tensor) -> torch.Tensor:          # [T, groups, in] -> [T, groups, out / groups]
        w = self.weight.view(self.groups, -1, x.shape[-1])
        return torch.einsum("tgi,goi->tgo", x, w)


class DSV4Attention(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx = arch, layer_idx
        self.kind = arch.layer_types[layer_idx] if arch.layer_types else "sliding_attention"
        a, std = arch, arch.initializer_range
        self.nh, self.D = a.num_attention_heads, a.head_dim
        self.q_a_proj = Linear(a.hidden_size, a.q_lora_rank, std=std, dtype=dtype, device=device)
        self.q_a_norm = RMSNorm(a.q_lora_rank, a.rms_norm_eps, dtype=dtype, device=device)
        self.q_b_proj = Linear(a.q_lora_rank, self.nh * self.D, std=std, dtype=dtype, device=device)
        self.kv_proj = Linear(a.hidden_size, self.D, std=std, dtype=dtype, device=device)
        self.kv_norm = RMSNorm(self.D, a.rms_norm_eps, dtype=dtype, device=device)
        self.o_a_proj = GroupedLinear(self.nh * self.D // a.o_groups, a.o_groups * a.o_lora_rank, a.o_groups, std,
                                      dtype=dtype, device=device)
        self.o_b_proj = Linear(a.o_groups * a.o_lora_rank, a.hidden_size, std=std, dtype=dtype, device=device)
        self.sinks = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32, device=device))
        self.compressor = self.indexer = None
        if self.kind == "compressed_sparse_attention":
            self.compressor = Compressor(a, self.D, a.csa_compress_rate, 2, dtype=dtype, device=device)
            self.indexer = LightningIndexer(a, dtype=dtype, device=device)
        elif self.kind == "heavily_compressed_attention":
            self.compressor = Compressor(a, self.D, a.hca_compress_rate, 1, dtype=dtype, device=device)
        from ..ops import inv_freq

        theta = a.rope_theta if self.kind == "sliding_attention" else a.compress_rope_theta
        self.register_buffer("inv_freq", inv_freq(a.qk_rope_head_dim, theta, device=device), persistent=False)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        a, T = self.arch, x.shape[0]
        ctx = packed_context(seq, a)
        q_res = self.q_a_norm(self.q_a_proj(x))
        q = unweighted_rms_norm(self.q_b_proj(q_res).view(T, self.nh, self.D), a.rms_norm_eps)
        q = rope_interleaved(q, seq.position_ids, self.inv_freq)
        kv = rope_interleaved(self.kv_norm(self.kv_proj(x)).view(T, 1, self.D), seq.position_ids, self.inv_freq)[:, 0]
        if seq.engine is not None:
            o = self._engine_attention(x, seq, q, kv, q_res)
            o = rope_interleaved(o, seq.position_ids, self.inv_freq, conj=True)
            return self.o_b_proj(self.o_a_proj(o.reshape(T, a.o_groups, -1)).flatten(1))
        indices, kv_buf = ctx["window"], kv
        if ctx.get("gather") is not None:          # context parallelism: all tokens' rows, slots in global numbering
            kv_buf = kv = ctx["gather"](kv)
        if self.compressor is not None:
            layout = ctx["layouts"][self.compressor.rate]
            entries = self.compressor.compress(x, layout, ctx.get("gather"))
            if self.indexer is not None:
                picks = self.indexer(x, q_res, seq, ctx)
            else:                     # every completed entry of the query's own document
                ready = self.compressor.readable_entries(seq.position_ids)[:, None]
                base = layout.first_entry_of_doc[ctx["doc"]][:, None]
                off = torch.arange(max(layout.max_per_doc, 1), device=x.device)[None, :]
                picks = torch.where(off < ready, base + off, torch.full_like(base + off, IGNORE_SLOT))
            kv_buf = torch.cat([kv, entries], dim=0)        # tokens first, this layer's entries after
            indices = torch.cat([indices, torch.where(picks >= 0, picks + kv.shape[0], picks)], dim=1)
        o = sparse_mla.slot_attention(q, kv_buf, indices, self.D ** -0.5, self.sinks)
        o = rope_interleaved(o, seq.position_ids, self.inv_freq, conj=True)      # values carried the keys' rotation
        g = self.o_a_proj(o.reshape(T, a.o_groups, -1)).flatten(1)
        return self.o_b_proj(g)


    def _engine_attention(self, x, seq: SeqInfo, q, kv, q_res) -> torch.Tensor:
        """Rollout engine: every sequence keeps its tokens' shared K / V rows, its completed entries and the
        projections of the tokens that unfinished entries still need (``engine/hybrid.py: RecurrentStep``)."""
        a, eng = self.arch, seq.engine
        outs = []
        back = torch.arange(a.sliding_window, device=x.device)
        for r, store, L in eng.sequences():
            kv_all = eng.append(store, (self.layer_idx, "kv"), kv[r], L)
            pos = seq.position_ids[r].long()
            win = pos[:, None] - back[None, :]                               # most recent token first
            indices = torch.where(win >= 0, win, torch.full_like(win, IGNORE_SLOT))
            kv_buf = kv_all
            if self.compressor is not None:
                entries = self.compressor.engine_entries(eng, store, (self.layer_idx, "cmp"), x[r], L)
                if self.indexer is not None:
                    picks = self.indexer.engine_picks(eng, store, self.layer_idx, x[r], q_res[r], pos, L)
                else:
                    ready = self.compressor.readable_entries(pos)[:, None]
                    off = torch.arange(max(entries.shape[0], 1), device=x.device)[None, :]
                    picks = torch.where(off < ready, off.expand(pos.shape[0], -1), torch.full_like(off, IGNORE_SLOT))
                kv_buf = torch.cat([kv_all, entries.to(kv_all.dtype)], dim=0)
                indices = torch.cat([indices, torch.where(picks >= 0, picks + kv_all.shape[0], picks)], dim=1)
            outs.append(sparse_mla.slot_attention(q[r], kv_buf, indices, self.D ** -0.5, self.sinks))
        return torch.cat(outs, 0)


# ---------------------------------------------------------------------- MoE
class DSV4Router(nn.Module):
    """``sqrt(softplus(logits))`` scores; top-k with a selection bias, or (hash layers) a frozen
    token-id -> experts table. Weights are always normalised over the selected experts."""

    def __init__(self, arch: ModelArch, is_hash: bool, dtype=None, device=None):
        super().__init__()
        self.arch, self.is_hash = arch, is_hash
        self.gate = Linear(arch.hidden_size, arch.num_experts, std=arch.initializer_range, dtype=dtype, device=device)
        if is_hash:
            self.register_buffer("tid2eid", torch.zeros(arch.vocab_size, arch.num_experts_per_tok, dtype=torch.long,
                                                        device=device))
            self.e_score_correction_bias = None
        else:
            self.register_buffer("e_score_correction_bias", torch.zeros(arch.num_experts, dtype=torch.float32,
                                                                        device=device))
        self.force_balanced = False

    def forward(self, x: torch.Tensor, forced: torch.Tensor | None = None, input_ids: torch.Tensor | None = None):
        a = self.arch
        scores = F.softplus(x.float() @ self.gate.weight.float().t()).sqrt()
        if forced is None and self.is_hash:
            if input_ids is None:
                raise ValueError("a hash-routed layer needs the token ids")
            forced = self.tid2eid[input_ids.reshape(-1)]
        if forced is not None:
            idx = forced.long()
        else:
            idx = (scores + self.e_score_correction_bias).topk(a.num_experts_per_tok, dim=1).indices
        w = scores.gather(1, idx)
        w = w / (w.sum(-1, keepdim=True) + 1e-20) * a.routed_scaling_factor
        counts = torch.bincount(idx.reshape(-1), minlength=a.num_experts).to(torch.int32)   # the plan kernel reads int32
        return idx.to(torch.int32).contiguous(), w, counts, scores


class DSV4MoE(MoE):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__(arch, layer_idx, dtype=dtype, device=device)
        self.is_hash = layer_idx < arch.num_hash_layers
        self.router = DSV4Router(arch, self.is_hash, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        T = x.shape[0]
        forced = seq.routed_experts[:, self.layer_idx, :] if seq.routed_experts is not None else None
        idx, w, counts, _ = self.router(x, forced, (seq.shared or {}).get("input_ids"))
        self.last_counts, self.last_topk = counts, idx
        if self.dispatcher is not None:
            y = self.dispatcher(self.experts, x, idx, w, counts)
        else:
            plan = moe_ops.build_plan(idx, counts, self.arch.num_experts)
            yp = self.experts(moe_ops.permute(x, plan), plan.block_expert, plan.expert_offset)
            y = moe_ops.combine(yp, w, plan, T)
        if self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y


class DSV4DecoderLayer(nn.Module):
    """Works on the stream tensor ``[T, hc, hidden]``."""

    def __init__(self, arch: ModelArch, layer_idx: int, attn_backend: str = "auto", dtype=None, device=None):
        super().__init__()
        self.attn_hc = HyperConnection(arch, dtype=dtype, device=device)
        self.ffn_hc = HyperConnection(arch, dtype=dtype, device=device)
        self.input_layernorm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)
        self.self_attn = DSV4Attention(arch, layer_idx, dtype=dtype, device=device)
        self.is_moe = arch.layer_is_moe(layer_idx)
        self.mlp = DSV4MoE(arch, layer_idx, dtype=dtype, device=device) if self.is_moe else DenseMLP(arch, dtype=dtype,
                                                                                                    device=device)

    def forward(self, streams: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        post, comb, x = self.attn_hc(streams)
        streams = HyperConnection.merge(streams, self.self_attn(self.input_layernorm(x), seq), post, comb)
        post, comb, x = self.ffn_hc(streams)
        x = self.post_attention_layernorm(x)
        m = self.mlp(x, seq) if self.is_moe else self.mlp(x)
        return HyperConnection.merge(streams, m, post, comb)
