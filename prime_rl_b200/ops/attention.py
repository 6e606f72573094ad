"""Variable-length (packed) causal attention.

Inputs are packed token-major tensors ``q [T, Hq, D]``, ``k/v [T, Hkv, D]`` with document
boundaries ``cu_seqlens`` (int32 ``[num_docs + 1]``): a token attends only to earlier
tokens of its own document, optionally inside a sliding window, optionally with a learnable
per-head sink logit that only takes probability mass (GPT-OSS).

Backends
--------
``tcgen05``            hand-written sm_100a kernel (``csrc/flash_attn.cu``) when built;
``flash_attention_2``  the flash-attn library (baseline arm, same call as the reference's
                       layers/attn.py:101-115);
``sdpa``               fp32 PyTorch reference with an explicit mask (CPU, oracles).
"""

from __future__ import annotations

import math

import torch


def attention_ref(q, k, v, cu_seqlens, *, causal=True, window=None, sinks=None, scale=None):
    """fp32 reference; O(T^2) memory, for tests and CPU runs."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf, kf, vf = q.float(), k.float(), v.float()
    rep = Hq // Hkv
    kf = kf.repeat_interleave(rep, dim=1)
    vf = vf.repeat_interleave(rep, dim=1)
    s = torch.einsum("thd,shd->hts", qf, kf) * scale
    pos = torch.arange(T, device=q.device)
    doc = torch.searchsorted(cu_seqlens[1:].to(torch.long).contiguous(), pos, right=True)
    mask = doc[:, None] == doc[None, :]
    if causal:
        mask &= pos[None, :] <= pos[:, None]
    if window is not None:
        mask &= pos[:, None] - pos[None, :] < window
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        sink = sinks.float().view(Hq, 1, 1).expand(Hq, T, 1)
        p = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :-1]
    else:
        p = torch.softmax(s, dim=-1)
    o = torch.einsum("hts,shd->thd", p, vf)
    return o.to(q.dtype)


# Which kernel computes the attention backward when the forward ran on the tcgen05 kernel:
# "tcgen05" (csrc/flash_attn_bwd.cu) or "flash_attention_2" (library).
BWD_BACKEND = "tcgen05"


def _fa2():
    from flash_attn.flash_attn_interface import _flash_attn_varlen_backward, _flash_attn_varlen_forward

    return _flash_attn_varlen_forward, _flash_attn_varlen_backward


def default_backend(device: torch.device) -> str:
    if device.type != "cuda":
        return "sdpa"
    from . import flash_native

    return "tcgen05" if flash_native.available() else "flash_attention_2"


class _FlashAttention(torch.autograd.Function):
    """Forward: the tcgen05 kernel (or the flash-attn library for shapes it does not cover).
    Backward: flash-attn library kernel on the saved (q, k, v, out, lse). ``cached`` carries
    (out, lse) computed by an earlier no-grad pass of the same layer (activation
    recomputation), in which case the forward launches nothing."""

    @staticmethod
    def forward(ctx, q, k, v, cu, max_seqlen, scale, window, backend, cached, store, q_offset=None, sinks=None):
        ws = (-1, -1) if window is None else (window - 1, 0)
        sinks32 = None if sinks is None else sinks.detach().float().contiguous()
        if cached is not None:
            out, lse = cached
        elif backend == "tcgen05":
            from . import flash_native

            out, lse = flash_native.flash_fwd(q, k, v, cu, scale=scale, window=window, q_offset=q_offset,
                                              sinks=sinks32)
        else:
            fwd, _ = _fa2()
            out, lse, _, _ = fwd(q, k, v, cu, cu, max_seqlen, max_seqlen, 0.0, scale, True, ws[0], ws[1], 0.0, None,
                                 False, None)
        if store is not None:
            store.append((out, lse))
        ctx.save_for_backward(q, k, v, out, lse, cu, sinks32)
        ctx.cfg = (max_seqlen, scale, ws, window, backend, q_offset)
        ctx.sink_dtype = None if sinks is None else sinks.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu, sinks32 = ctx.saved_tensors
        max_seqlen, scale, ws, window, backend, q_offset = ctx.cfg
        dsinks = None
        if sinks32 is not None:
            # d sink_h = - sum_t p_sink[h, t] * <dO[t, h], O[t, h]>, p_sink = exp(sink_h - lse[h, t]); dq / dk / dv
            # follow from the saved lse (which contains the sink) like without one
            delta = (dout.float() * out.float()).sum(-1)                         # [T, Hq]
            p_sink = torch.exp(sinks32.view(-1, 1) - lse)                        # [Hq, T]
            dsinks = -(p_sink * delta.t()).sum(-1).to(ctx.sink_dtype)
        if backend == "tcgen05" and BWD_BACKEND == "tcgen05":
            from . import flash_native

            if flash_native.bwd_available():
                dq, dk, dv = flash_native.flash_bwd(dout, q, k, v, out, lse, cu, scale=scale, window=window,
                                                    q_offset=q_offset)
                return dq, dk, dv, None, None, None, None, None, None, None, None, dsinks
        assert sinks32 is None, "attention sinks need the tcgen05 kernels"
        assert q_offset is None, "query slices need the tcgen05 kernels"
        _, bwd = _fa2()
        dq, dk, dv = torch.empty_like(q), torch.empty(k.shape, dtype=k.dtype, device=k.device), \
            torch.empty(v.shape, dtype=v.dtype, device=v.device)
        bwd(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, cu, cu, max_seqlen, max_seqlen, 0.0, scale, True, ws[0],
            ws[1], 0.0, None, False, None)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


def attention(q, k, v, cu_seqlens, max_seqlen: int, *, causal: bool = True, window: int | None = None,
              sinks: torch.Tensor | None = None, scale: float | None = None, backend: str = "auto",
              cache: dict | None = None, cache_key=None, q_offset: int | None = None):
    """``cache`` (a dict owned by the caller) lets an activation-recomputation pass reuse the
    attention output of the first pass of the same layer: a call whose ``cache_key`` is absent
    computes and stores ``(out, lse)``; the next call with that key consumes the entry and
    launches no forward kernel. ``q_offset`` (context parallelism): ``q`` holds only the global
    rows ``[q_offset, q_offset + len(q))`` while k / v / cu_seqlens cover the whole sequence."""
    if backend in ("auto", None, "flash_attention_3", "flash_attention_4"):
        backend = default_backend(q.device)
    fast = q.is_cuda and causal and q.dtype == torch.bfloat16 and backend != "sdpa"
    if fast and sinks is not None and not (backend == "tcgen05" and q.shape[-1] == 128):
        fast = False                     # the library kernels have no sink column
    if not fast:
        return attention_ref(q, k, v, cu_seqlens, causal=causal, window=window, sinks=sinks, scale=scale)
    if backend == "tcgen05" and q.shape[-1] != 128:
        backend = "flash_attention_2"
    if q_offset is not None and backend != "tcgen05":
        raise NotImplementedError("query-slice attention needs head_dim 128 and the tcgen05 backend")
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    cached = store = None
    if cache is not None:
        cached = cache.pop(cache_key, None)
        if cached is None:
            store = []
    out = _FlashAttention.apply(q, k, v, cu_seqlens, max_seqlen, scale, window, backend, cached, store, q_offset,
                                sinks)
    if store:
        cache[cache_key] = store.pop()
    return out
