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
                                      out.data_ptr(), rt.ptr(rstd), None, T, Hh, D, x.stride(0), out.stride(0),
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
                                      float(ctx.eps), 1, rt.stream_ptr(x.device))
        rt.check(rc, "prb_qknorm_rope(bwd)")
        # dx is written with x's pitch
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
