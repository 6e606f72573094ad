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


_flash = None


def _flash_attn():
    global _flash
    if _flash is None:
        from flash_attn import flash_attn_varlen_func

        _flash = flash_attn_varlen_func
    return _flash


def default_backend(device: torch.device) -> str:
    if device.type != "cuda":
        return "sdpa"
    try:
        from . import flash_native

        if flash_native.available():
            return "tcgen05"
    except Exception:
        pass
    return "flash_attention_2"


def attention(q, k, v, cu_seqlens, max_seqlen: int, *, causal: bool = True, window: int | None = None,
              sinks: torch.Tensor | None = None, scale: float | None = None, backend: str = "auto"):
    if backend in ("auto", None):
        backend = default_backend(q.device)
    if backend in ("flash_attention_3", "flash_attention_4"):
        backend = default_backend(q.device)
    if backend == "tcgen05" and sinks is None and q.shape[-1] == 128 and q.dtype == torch.bfloat16:
        from . import flash_native

        return flash_native.flash_attn_varlen(q, k, v, cu_seqlens, max_seqlen, causal=causal, window=window,
                                              scale=scale)
    if backend in ("tcgen05", "flash_attention_2") and q.is_cuda and sinks is None:
        ws = (-1, -1) if window is None else (window - 1, 0)
        return _flash_attn()(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, softmax_scale=scale,
                             causal=causal, window_size=ws)
    return attention_ref(q, k, v, cu_seqlens, causal=causal, window=window, sinks=sinks, scale=scale)
