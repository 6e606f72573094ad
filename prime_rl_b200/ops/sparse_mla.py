"""DeepSeek-style sparse attention (DSA) over a compressed multi-head-latent KV stream.

Two steps per layer:

``dsa_indexer_topk``   a light "indexer" scores every (query, key) pair of a document with
    ``sum_h w[t, h] * relu(q_idx[t, h] . k_idx[s])``, restricted to the window ``[ks[t], ke[t])``
    (document start .. causal end), and keeps the ``topk`` best keys per query. Slots that cannot
    be filled carry the sentinel index ``S`` (= number of keys). No gradient flows through the
    selection.
``sparse_mla_attention``   every query attends only to its selected rows of the single shared
    latent KV stream ``kv [S, d_latent + d_rope]``: scores use all ``d_latent + d_rope`` channels,
    values are the first ``d_v = d_latent`` channels of the same rows (weight absorption moves the
    per-head up-projections outside of the attention).

Queries are processed in blocks so that the gathered KV rows of a block stay within a fixed
budget; the backward pass comes from autograd (a scatter-add into the KV stream).

The reference implements these as a Triton fp8 scoring kernel plus ``torch.topk``
(src/prime_rl/trainer/models/kernels/fp8_indexer.py:91-238) and TileLang kernels
(kernels/sparse_mla_fwd.py:23-186, sparse_mla_bwd.py:21-277).
"""

from __future__ import annotations

import torch


@torch.no_grad()
def dsa_indexer_topk(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor,
                     topk: int, block: int = 1024) -> torch.Tensor:
    """``q_idx [T, Hi, Di]``, ``k_idx [S, Di]``, ``w [T, Hi]``, ``ks, ke [T]`` -> int32 ``[T, topk]``."""
    T, S = q_idx.shape[0], k_idx.shape[0]
    kk = min(topk, S)
    out = torch.full((T, topk), S, dtype=torch.int32, device=q_idx.device)
    cols = torch.arange(S, device=q_idx.device)
    kT = k_idx.float().t()
    for t0 in range(0, T, block):
        t1 = min(T, t0 + block)
        s = torch.relu(torch.einsum("thd,ds->ths", q_idx[t0:t1].float(), kT))
        logits = (s * w[t0:t1].float().unsqueeze(-1)).sum(1)
        valid = (cols[None, :] >= ks[t0:t1, None]) & (cols[None, :] < ke[t0:t1, None])
        logits = logits.masked_fill(~valid, float("-inf"))
        idx = logits.topk(kk, dim=-1).indices
        ok = torch.gather(valid, 1, idx)
        out[t0:t1, :kk] = torch.where(ok, idx, torch.full_like(idx, S)).to(torch.int32)
    return out


def sparse_mla_attention(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, scale: float, d_v: int,
                         rows_budget: int = 1 << 18) -> torch.Tensor:
    """``q [T, H, Dqk]``, ``kv [S, Dqk]``, ``indices [T, topk]`` (sentinel ``S`` = empty slot) ->
    ``[T, H, d_v]`` in the dtype of ``q``. A query without any valid slot returns zeros."""
    T, H, Dqk = q.shape
    S = kv.shape[0]
    topk = indices.shape[1]
    kv_pad = torch.cat([kv, kv.new_zeros(1, Dqk)], dim=0)           # row S = the sentinel
    block = max(1, rows_budget // max(topk, 1))
    outs = []
    for t0 in range(0, T, block):
        t1 = min(T, t0 + block)
        idx = indices[t0:t1].long()
        g = kv_pad[idx]                                               # [b, topk, Dqk]
        s = torch.einsum("bhd,bkd->bhk", q[t0:t1].float(), g.float()) * scale
        valid = (idx < S).unsqueeze(1)
        s = s.masked_fill(~valid, float("-inf"))
        m = s.amax(-1, keepdim=True)
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = (s - m).exp()
        den = p.sum(-1, keepdim=True).clamp_min(1e-30)
        o = torch.einsum("bhk,bkd->bhd", p / den, g[..., :d_v].float())
        outs.append(o.to(q.dtype))
    return torch.cat(outs, dim=0)


def sparse_mla_attention_ref(q, kv, indices, scale, d_v) -> torch.Tensor:
    """Dense masked attention with the same selection (fp32), for tests."""
    T, H, Dqk = q.shape
    S = kv.shape[0]
    mask = torch.zeros(T, S + 1, dtype=torch.bool, device=q.device)
    mask.scatter_(1, indices.long(), True)
    mask = mask[:, :S]
    s = torch.einsum("thd,sd->ths", q.float(), kv.float()) * scale
    s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.where(mask.any(-1)[:, None, None], p, torch.zeros_like(p))
    return torch.einsum("ths,sd->thd", p, kv[:, :d_v].float())
