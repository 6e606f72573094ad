"""Gated activations (``csrc/elementwise.cu``): SwiGLU, clamped SwiGLU (GPT-OSS), ReLU^2."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _runtime as rt

SWIGLU, SWIGLU_CLAMPED, RELU2, SILU_CLAMPED = 0, 1, 2, 3    # SILU_CLAMPED: silu(min(g, L)) * clamp(u, -L, L) (DeepSeek-V4)


def glu_ref(g, u, act=SWIGLU, limit=7.0, alpha=1.702):
    gf = g.float()
    if act == SWIGLU:
        y = F.silu(gf) * u.float()
    elif act == SWIGLU_CLAMPED:
        gc = gf.clamp(max=limit)
        uc = u.float().clamp(-limit, limit)
        y = gc * torch.sigmoid(alpha * gc) * (uc + 1.0)
    elif act == SILU_CLAMPED:
        y = F.silu(gf.clamp(max=limit)) * u.float().clamp(-limit, limit)
    else:
        y = F.relu(gf) ** 2
    return y.to(g.dtype)


class _GLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act, limit, alpha):
        # gu: [rows, 2*I] = [gate | up] (or [rows, I] for ReLU^2)
        rows = gu.shape[0]
        I = gu.shape[1] if act == RELU2 else gu.shape[1] // 2
        y = torch.empty(rows, I, dtype=gu.dtype, device=gu.device)
        g_ptr = gu.data_ptr()
        u_ptr = g_ptr + I * gu.element_size()
        rc = rt.lib().prb_glu_fwd(g_ptr, u_ptr, y.data_ptr(), rows, I, gu.stride(0), y.stride(0), act,
                                  float(limit), float(alpha), rt.stream_ptr(gu.device))
        rt.check(rc, "prb_glu_fwd")
        ctx.save_for_backward(gu)
        ctx.cfg = (act, limit, alpha, I)
        return y

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        act, limit, alpha, I = ctx.cfg
        dy = dy.contiguous()
        dgu = torch.empty_like(gu)
        g_ptr = gu.data_ptr()
        u_ptr = g_ptr + I * gu.element_size()
        dg_ptr = dgu.data_ptr()
        du_ptr = dg_ptr + I * gu.element_size()
        rc = rt.lib().prb_glu_bwd(dy.data_ptr(), g_ptr, u_ptr, dg_ptr, du_ptr, gu.shape[0], I, gu.stride(0),
                                  dy.stride(0), dgu.stride(0), act, float(limit), float(alpha),
                                  rt.stream_ptr(gu.device))
        rt.check(rc, "prb_glu_bwd")
        return dgu, None, None, None


def glu_rowmask(gate_up: torch.Tensor, row_valid: torch.Tensor, act: int = SWIGLU, limit: float = 7.0,
                alpha: float = 1.702) -> torch.Tensor:
    """Inference-only ``glu`` over the padded row space of grouped experts: rows with ``row_valid < 0``
    (int32 per row) are neither read nor written, their outputs stay uninitialised."""
    rows = gate_up.shape[0]
    I = gate_up.shape[1] if act == RELU2 else gate_up.shape[1] // 2
    assert gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous() and I % 8 == 0
    assert act != SILU_CLAMPED and row_valid.dtype == torch.int32 and row_valid.numel() >= rows
    y = torch.empty(rows, I, dtype=gate_up.dtype, device=gate_up.device)
    g_ptr = gate_up.data_ptr()
    rc = rt.lib().prb_glu_fwd_rowmask(g_ptr, g_ptr + I * gate_up.element_size(), y.data_ptr(), rows, I, gate_up.stride(0),
                                      y.stride(0), act, float(limit), float(alpha), row_valid.data_ptr(),
                                      rt.stream_ptr(gate_up.device))
    rt.check(rc, "prb_glu_fwd_rowmask")
    return y


def glu(gate_up: torch.Tensor, act: int = SWIGLU, limit: float = 7.0, alpha: float = 1.702) -> torch.Tensor:
    """``gate_up`` holds ``[gate | up]`` along the last dim (just ``gate`` for ReLU^2)."""
    shape = gate_up.shape
    I = shape[-1] if act == RELU2 else shape[-1] // 2
    if act != SILU_CLAMPED and gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and I % 8 == 0:
        gu2 = gate_up.reshape(-1, shape[-1])
        if not gu2.is_contiguous():
            gu2 = gu2.contiguous()
        return _GLU.apply(gu2, act, limit, alpha).reshape(*shape[:-1], I)
    if act == RELU2:
        return glu_ref(gate_up, None, act)
    g, u = gate_up[..., :I], gate_up[..., I:]
    return glu_ref(g, u, act, limit, alpha)
