"""Fused per-head RMSNorm + rotary embedding (``csrc/norm_rope.cu``).

The rotation is the half-split form used by Llama/Qwen: with ``x = (x1, x2)`` split at
``D/2``, ``y = (x1 cos - x2 sin, x2 cos + x1 sin)`` and angle ``pos * inv_freq[i]``.
"""

from __future__ import annotations

import torch

from . import _runtime as rt


def inv_freq(head_dim: int, theta: float, device=None, rotary_dim: int | None = None) -> torch.Tensor:
    rd = rotary_dim or head_dim
    return 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32, device=device) / rd))


def qknorm_rope_ref(x, w, pos, inv_f, eps):
    """x: [T, heads, D]; w: [D] or None; pos: [T]; inv_f: [D/2]."""
    T, Hh, D = x.shape
    xf = x.float()
    if w is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        xf = xf.to(x.dtype).float()
    rd = inv_f.numel() * 2
    ang = pos.float()[:, None] * inv_f.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xr, xp = xf[..., :rd], xf[..., rd:]
    x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
    y = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, xp], dim=-1)
    return y.to(x.dtype)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, pos, inv_f, eps):
        T, Hh, D = x.shape
        assert x.stride(2) == 1 and x.stride(1) == D
        out = torch.empty(T, Hh, D, dtype=x.dtype, device=x.device)
        rstd = torch.empty(T * Hh, dtype=torch.float32, device=x.device) if w is not None else None
        rc = rt.lib().prb_qknorm_rope(x.data_ptr(), None, rt.ptr(w), pos.data_ptr(), inv_f.data_ptr(),
                                      out.data_ptr(), rt.ptr(rstd), None, T, Hh, D, x.stride(0), out.stride(0), 0,
                                      float(eps), 0, rt.stream_ptr(x.device))
        rt.check(rc, "prb_qknorm_rope")
        ctx.save_for_backward(x, w, pos, inv_f, rstd)
        ctx.eps = eps
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, pos, inv_f, rstd = ctx.saved_tensors
        T, Hh, D = x.shape
        dy = dy.contiguous()
        dx = torch.empty(T, Hh, D, dtype=x.dtype, device=x.device)
        need_dw = w is not None and ctx.needs_input_grad[1]
        dw = torch.zeros(D, dtype=torch.float32, device=x.device) if need_dw else None
        rc = rt.lib().prb_qknorm_rope(x.data_ptr(), dy.data_ptr(), rt.ptr(w), pos.data_ptr(), inv_f.data_ptr(),
                                      dx.data_ptr(), rt.ptr(rstd), rt.ptr(dw), T, Hh, D, x.stride(0), dy.stride(0),
                                      dx.stride(0), float(ctx.eps), 1, rt.stream_ptr(x.device))
        rt.check(rc, "prb_qknorm_rope(bwd)")
        return dx, (dw.to(w.dtype) if need_dw else None), None, None, None


def qknorm_rope(x: torch.Tensor, w: torch.Tensor | None, pos: torch.Tensor, inv_f: torch.Tensor,
                eps: float = 1e-6) -> torch.Tensor:
    """x: [T, heads, D] (token pitch may exceed heads*D, e.g. a slice of a packed qkv
    projection); returns a contiguous [T, heads, D]."""
    D = x.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and D in (64, 128, 256) and inv_f.numel() * 2 == D
            and (w is None or w.dtype == torch.bfloat16)):
        if x.stride(2) != 1 or x.stride(1) != D:
            x = x.contiguous()
        return _QKNormRope.apply(x, w, pos.to(torch.int32), inv_f, eps)
    return qknorm_rope_ref(x, w, pos, inv_f, eps)


class _QKVNormRope(torch.autograd.Function):
    """Splits a packed qkv projection, applies per-head RMSNorm + RoPE to q and k, and in
    backward writes dq / dk / dv straight into one ``[T, W]`` gradient (no slice-backward
    zero fills and adds)."""

    @staticmethod
    def forward(ctx, qkv, qw, kw, pos, inv_f, eps, nq, nkv, D):
        T, W = qkv.shape
        qd, kd = nq * D, nkv * D
        q = torch.empty(T, nq, D, dtype=qkv.dtype, device=qkv.device)
        k = torch.empty(T, nkv, D, dtype=qkv.dtype, device=qkv.device)
        has_norm = qw is not None
        rq = torch.empty(T * nq, dtype=torch.float32, device=qkv.device) if has_norm else None
        rk = torch.empty(T * nkv, dtype=torch.float32, device=qkv.device) if has_norm else None
        es = qkv.element_size()
        st = rt.stream_ptr(qkv.device)
        rc = rt.lib().prb_qknorm_rope(qkv.data_ptr(), None, rt.ptr(qw), pos.data_ptr(), inv_f.data_ptr(),
                                      q.data_ptr(), rt.ptr(rq), None, T, nq, D, W, qd, 0, float(eps), 0, st)
        rt.check(rc, "prb_qknorm_rope(q)")
        rc = rt.lib().prb_qknorm_rope(qkv.data_ptr() + qd * es, None, rt.ptr(kw), pos.data_ptr(), inv_f.data_ptr(),
                                      k.data_ptr(), rt.ptr(rk), None, T, nkv, D, W, kd, 0, float(eps), 0, st)
        rt.check(rc, "prb_qknorm_rope(k)")
        v = qkv[:, qd + kd:].view(T, nkv, D)
        ctx.save_for_backward(qkv, qw, kw, pos, inv_f, rq, rk)
        ctx.cfg = (eps, nq, nkv, D)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, qw, kw, pos, inv_f, rq, rk = ctx.saved_tensors
        eps, nq, nkv, D = ctx.cfg
        T, W = qkv.shape
        qd, kd = nq * D, nkv * D
        es = qkv.element_size()
        dqkv = torch.empty_like(qkv)
        dq, dk = dq.contiguous(), dk.contiguous()
        need_w = qw is not None and (ctx.needs_input_grad[1] or ctx.needs_input_grad[2])
        dqw = torch.zeros(D, dtype=torch.float32, device=qkv.device) if need_w else None
        dkw = torch.zeros(D, dtype=torch.float32, device=qkv.device) if need_w else None
        st = rt.stream_ptr(qkv.device)
        rc = rt.lib().prb_qknorm_rope(qkv.data_ptr(), dq.data_ptr(), rt.ptr(qw), pos.data_ptr(), inv_f.data_ptr(),
                                      dqkv.data_ptr(), rt.ptr(rq), rt.ptr(dqw), T, nq, D, W, qd, W, float(eps), 1, st)
        rt.check(rc, "prb_qknorm_rope(dq)")
        rc = rt.lib().prb_qknorm_rope(qkv.data_ptr() + qd * es, dk.data_ptr(), rt.ptr(kw), pos.data_ptr(),
                                      inv_f.data_ptr(), dqkv.data_ptr() + qd * es, rt.ptr(rk), rt.ptr(dkw), T, nkv, D,
                                      W, kd, W, float(eps), 1, st)
        rt.check(rc, "prb_qknorm_rope(dk)")
        dqkv[:, qd + kd:].copy_(dv.reshape(T, kd))
        return (dqkv, dqw.to(qw.dtype) if need_w else None, dkw.to(kw.dtype) if need_w else None, None, None, None,
                None, None, None)


def qkv_norm_rope(qkv: torch.Tensor, qw, kw, pos, inv_f, eps: float, nq: int, nkv: int, D: int):
    """qkv: [T, (nq + 2 nkv) * D] -> (q [T, nq, D], k [T, nkv, D], v [T, nkv, D])."""
    T = qkv.shape[0]
    qd, kd = nq * D, nkv * D
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and D in (64, 128, 256) and inv_f.numel() * 2 == D
            and qkv.is_contiguous() and (qw is None or qw.dtype == torch.bfloat16)):
        return _QKVNormRope.apply(qkv, qw, kw, pos.to(torch.int32), inv_f, eps, nq, nkv, D)
    q = qkv[:, :qd].view(T, nq, D)
    k = qkv[:, qd:qd + kd].view(T, nkv, D)
    v = qkv[:, qd + kd:].view(T, nkv, D)
    return qknorm_rope(q, qw, pos, inv_f, eps), qknorm_rope(k, kw, pos, inv_f, eps), v


def qkv_rope_to_cache(qkv: torch.Tensor, qw, kw, pos, inv_f, eps: float, nq: int, nkv: int, D: int,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor, want_kv: bool = True):
    """Inference-only: ``qkv_norm_rope`` plus the write of K / V into the paged cache
    (``k_cache`` / ``v_cache``: [pages, page_size, nkv, D]; ``slots``: int64 [T] rows of the flattened cache)
    in ONE launch. Returns (q, k, v); k and v are None unless ``want_kv`` (a decode step reads them
    from the cache only). Falls back to the separate ops where the kernel does not apply."""
    T = qkv.shape[0]
    fused = (qkv.is_cuda and qkv.dtype == torch.bfloat16 and D in (64, 128, 256) and inv_f.numel() * 2 == D
             and qkv.is_contiguous() and (qw is None or qw.dtype == torch.bfloat16) and k_cache.dtype == torch.bfloat16
             and k_cache.is_contiguous() and v_cache.is_contiguous() and slots.dtype == torch.int64
             and not torch.is_grad_enabled())
    if not fused:
        q, k, v = qkv_norm_rope(qkv, qw, kw, pos, inv_f, eps, nq, nkv, D)
        kf, vf = k_cache.view(-1, nkv, D), v_cache.view(-1, nkv, D)
        kf.index_copy_(0, slots, k.to(kf.dtype))
        vf.index_copy_(0, slots, v.to(vf.dtype))
        return q, k, v
    pos32 = pos.to(torch.int32)
    q = torch.empty(T, nq, D, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, nkv, D, dtype=qkv.dtype, device=qkv.device) if want_kv else None
    v = torch.empty_like(k) if want_kv else None
    rc = rt.lib().prb_qkv_rope_cache(qkv.data_ptr(), rt.ptr(qw), rt.ptr(kw), pos32.data_ptr(),
                                     inv_f.data_ptr(), slots.data_ptr(), q.data_ptr(), rt.ptr(k), rt.ptr(v),
                                     k_cache.data_ptr(), v_cache.data_ptr(), T, nq, nkv, D, float(eps),
                                     rt.stream_ptr(qkv.device))
    rt.check(rc, "prb_qkv_rope_cache")
    return q, k, v
