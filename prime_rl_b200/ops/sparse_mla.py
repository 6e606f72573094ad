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

On a GPU, bf16 inputs with the DeepSeek / GLM latent shape (512 + 64 channels, at most 128 heads)
run the tcgen05 forward kernel (``csrc/sparse_mla.cu``), which never materialises the gathered
rows; its backward recomputes the probabilities from the saved log-sum-exp block by block in
PyTorch. Everything else takes the PyTorch path: queries are processed in blocks so that the
gathered KV rows of a block stay within a fixed budget, and the backward pass comes from
autograd (a scatter-add into the KV stream).

The reference implements these as a Triton fp8 scoring kernel plus ``torch.topk``
(src/prime_rl/trainer/models/kernels/fp8_indexer.py:91-238) and TileLang kernels
(kernels/sparse_mla_fwd.py:23-186, sparse_mla_bwd.py:21-277).
"""

from __future__ import annotations

import torch

from . import _runtime as rt


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
        # The ReLU makes exact ties (several keys at 0) common. A stable sort breaks them towards the earlier key, so
        # that the selection of a query does not depend on how many keys follow it in the call: the rollout engine
        # (keys up to the query) and the trainer (the whole packed sequence) then pick the same keys.
        idx = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :kk]
        ok = torch.gather(valid, 1, idx)
        out[t0:t1, :kk] = torch.where(ok, idx, torch.full_like(idx, S)).to(torch.int32)
    return out


class _SparseMLAKernel(torch.autograd.Function):
    """tcgen05 forward; backward recomputed in blocks of queries from (out, lse)."""

    @staticmethod
    def forward(ctx, q, kv, indices, scale, rows_budget):
        T, H, Dqk = q.shape
        S = kv.shape[0]
        dev = q.device
        q, kv = q.contiguous(), kv.contiguous()
        idx = indices.to(torch.int32)
        pad = (-idx.shape[1]) % 64
        if pad:
            idx = torch.nn.functional.pad(idx, (0, pad), value=S)
        idx = idx.contiguous()
        out = torch.empty(T, H, 512, dtype=torch.bfloat16, device=dev)
        lse = torch.empty(T, H, dtype=torch.float32, device=dev)
        rt.check(rt.lib().prb_sparse_mla_fwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                             T, H, S, idx.shape[1], float(scale), rt.status_tensor(dev).data_ptr(),
                                             rt.stream_ptr(dev)), "prb_sparse_mla_fwd")
        ctx.save_for_backward(q, kv, idx, out, lse)
        ctx.scale, ctx.rows_budget = scale, rows_budget
        return out

    @staticmethod
    def backward(ctx, dout):
        q, kv, idx, out, lse = ctx.saved_tensors
        T, H, Dqk = q.shape
        S, scale = kv.shape[0], ctx.scale
        topk = idx.shape[1]
        kv_pad = torch.cat([kv, kv.new_zeros(1, Dqk)], dim=0)
        dq = torch.empty_like(q)
        dkv = torch.zeros(S + 1, Dqk, dtype=torch.float32, device=q.device)
        block = max(1, ctx.rows_budget // topk)
        dout = dout.contiguous()
        for t0 in range(0, T, block):
            t1 = min(T, t0 + block)
            ix = idx[t0:t1].long().clamp(0, S)
            g = kv_pad[ix]                                               # [b, topk, Dqk] bf16
            s = torch.einsum("bhd,bkd->bhk", q[t0:t1], g).float() * scale
            lse_b = lse[t0:t1].unsqueeze(-1)
            p = torch.where((ix < S).unsqueeze(1) & torch.isfinite(lse_b), (s - lse_b).exp(), torch.zeros_like(s))
            do = dout[t0:t1]
            dp = torch.einsum("bhd,bkd->bhk", do, g[..., :512]).float()
            delta = (do.float() * out[t0:t1].float()).sum(-1, keepdim=True)
            ds = (p * (dp - delta) * scale).to(q.dtype)
            dq[t0:t1] = torch.einsum("bhk,bkd->bhd", ds, g)
            dg = torch.einsum("bhk,bhd->bkd", ds, q[t0:t1]).float()
            dg[..., :512] += torch.einsum("bhk,bhd->bkd", p.to(q.dtype), do).float()
            dkv.index_add_(0, ix.reshape(-1), dg.reshape(-1, Dqk))
        return dq, dkv[:S].to(kv.dtype), None, None, None


def _kernel_eligible(q, kv, indices, d_v) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and q.shape[-1] == 576
            and d_v == 512 and q.shape[1] <= 128 and kv.shape[-1] == 576)


def sparse_mla_attention(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, scale: float, d_v: int,
                         rows_budget: int = 1 << 18) -> torch.Tensor:
    """``q [T, H, Dqk]``, ``kv [S, Dqk]``, ``indices [T, topk]`` (sentinel ``S`` = empty slot) ->
    ``[T, H, d_v]`` in the dtype of ``q``. A query without any valid slot returns zeros."""
    if _kernel_eligible(q, kv, indices, d_v):
        return _SparseMLAKernel.apply(q, kv, indices, scale, rows_budget)
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


def slot_attention(q: torch.Tensor, kv_buf: torch.Tensor, indices: torch.Tensor, scale: float,
                   sinks: torch.Tensor | None = None, rows_budget: int = 1 << 18) -> torch.Tensor:
    """Shared-KV attention over explicit slots (DeepSeek-V4): query ``t`` attends to the rows
    ``indices[t, :]`` of ``kv_buf [N, D]`` (negative or out-of-range = empty slot); a row is key and
    value at once; ``sinks [H]`` adds one learnable logit per head to the softmax denominator
    (it takes probability mass but contributes no value). ``q [T, H, D]`` -> ``[T, H, D]``.

    Same contract as the reference's ``dsv4_sparse_attn``
    (src/prime_rl/trainer/models/kernels/deepseek_v4/dsv4_sparse_attn.py:84-222)."""
    T, H, D = q.shape
    N = kv_buf.shape[0]
    slots = indices.shape[1]
    kv_pad = torch.cat([kv_buf, kv_buf.new_zeros(1, D)], dim=0)
    block = max(1, rows_budget // max(slots, 1))
    outs = []
    for t0 in range(0, T, block):
        t1 = min(T, t0 + block)
        idx = indices[t0:t1].long()
        idx = torch.where((idx < 0) | (idx >= N), torch.full_like(idx, N), idx)
        g = kv_pad[idx]                                               # [b, slots, D]
        s = torch.einsum("bhd,bkd->bhk", q[t0:t1].float(), g.float()) * scale
        s = s.masked_fill((idx == N).unsqueeze(1), float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.float()[None, :, None].expand(t1 - t0, H, 1)], dim=-1)
        m = s.amax(-1, keepdim=True)
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = (s - m).exp()
        p = p / p.sum(-1, keepdim=True).clamp_min(1e-30)
        if sinks is not None:
            p = p[..., :-1]
        outs.append(torch.einsum("bhk,bkd->bhd", p, g.float()).to(q.dtype))
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
