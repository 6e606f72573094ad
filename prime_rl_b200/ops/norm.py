"""RMSNorm (optionally fused with the residual add) — kernels in ``csrc/norm_rope.cu``."""

from __future__ import annotations

import torch

from . import _runtime as rt


def rms_norm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1])
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = rt.lib().prb_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), None, rstd.data_ptr(),
                                      rows, cols, float(eps), rt.stream_ptr(x.device))
        rt.check(rc, "prb_rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = dy.reshape(rows, cols)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        need_dw = ctx.needs_input_grad[1]
        dw = dwp = None
        if need_dw:
            parts = rt.lib().prb_rmsnorm_bwd_parts(rows)
            dwp = torch.empty(parts, cols, dtype=torch.float32, device=x2.device)
            dw = torch.empty(cols, dtype=torch.float32, device=x2.device)
        rc = rt.lib().prb_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                      dx.data_ptr(), rt.ptr(dwp), rt.ptr(dw), 0, rows, cols,
                                      rt.stream_ptr(x2.device))
        rt.check(rc, "prb_rmsnorm_bwd")
        return dx.reshape(ctx.shape), (dw.to(w.dtype) if need_dw else None), None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192:
        if not x.is_contiguous():
            x = x.contiguous()
        return _RMSNorm.apply(x, w, eps)
    return rms_norm_ref(x, w, eps)


class _AddRMSNorm(torch.autograd.Function):
    """h = x + residual (stored bf16); y = rmsnorm(h) * w. Returns (y, h)."""

    @staticmethod
    def forward(ctx, x, residual, w, eps):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, x.shape[-1])
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        h = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = rt.lib().prb_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), y.data_ptr(), h.data_ptr(),
                                      rstd.data_ptr(), rows, cols, float(eps), rt.stream_ptr(x.device))
        rt.check(rc, "prb_rmsnorm_fwd")
        ctx.save_for_backward(h, w, rstd)
        ctx.shape = x.shape
        return y.reshape(x.shape), h.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        rows, cols = h.shape
        dy2 = dy.reshape(rows, cols).contiguous()
        dh2 = dh.reshape(rows, cols).contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        need_dw = ctx.needs_input_grad[2]
        dw = dwp = None
        if need_dw:
            parts = rt.lib().prb_rmsnorm_bwd_parts(rows)
            dwp = torch.empty(parts, cols, dtype=torch.float32, device=h.device)
            dw = torch.empty(cols, dtype=torch.float32, device=h.device)
        rc = rt.lib().prb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), rt.ptr(dh2),
                                      dx.data_ptr(), rt.ptr(dwp), rt.ptr(dw), 0, rows, cols,
                                      rt.stream_ptr(h.device))
        rt.check(rc, "prb_rmsnorm_bwd")
        dx = dx.reshape(ctx.shape)
        return dx, dx, (dw.to(w.dtype) if need_dw else None), None


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """Returns ``(rmsnorm(x + residual) * w, x + residual)``."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192:
        return _AddRMSNorm.apply(x.contiguous(), residual.contiguous(), w, eps)
    h = x + residual
    return rms_norm_ref(h, w, eps), h
