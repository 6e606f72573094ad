"""Flat-buffer fused AdamW and gradient-norm clipping (``csrc/elementwise.cu``)."""

from __future__ import annotations

import math

import torch

from . import _runtime as rt


def adamw_ref(p, m, v, g, *, lr, b1, b2, eps, wd, step, grad_scale=1.0):
    g = g.float() * grad_scale
    bc1 = 1 - b1 ** step
    bc2 = 1 - b2 ** step
    p.mul_(1 - lr * wd)
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p.addcdiv_(m, denom, value=-lr / bc1)


def sumsq(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x^2); ``out`` is fp32 [1] on the same device."""
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous():
        rc = rt.lib().prb_sumsq(x.data_ptr(), x.numel(), int(x.dtype == torch.bfloat16), out.data_ptr(),
                                rt.stream_ptr(x.device))
        rt.check(rc, "prb_sumsq")
    else:
        out += x.float().pow(2).sum()


def clip_coef(sumsq_t: torch.Tensor, max_norm: float):
    """Returns (coef [1], norm [1]) on device, no host synchronisation."""
    if sumsq_t.is_cuda:
        coef = torch.empty(1, dtype=torch.float32, device=sumsq_t.device)
        norm = torch.empty(1, dtype=torch.float32, device=sumsq_t.device)
        rc = rt.lib().prb_clip_coef(sumsq_t.data_ptr(), float(max_norm), coef.data_ptr(), norm.data_ptr(),
                                    rt.stream_ptr(sumsq_t.device))
        rt.check(rc, "prb_clip_coef")
        return coef, norm
    norm = sumsq_t.sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
    return coef, norm


def adamw_flat(p, m, v, g, p_lowp, hyper, *, b1, b2, eps, wd, grad_scale=1.0, clip=None) -> None:
    """One launch over a flat fp32 master buffer. ``hyper`` = device fp32 [lr, 1-b1^t, sqrt(1-b2^t)]."""
    assert p.is_cuda
    rc = rt.lib().prb_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                            rt.ptr(p_lowp), p.numel(), hyper.data_ptr(), float(b1), float(b2), float(eps), float(wd),
                            float(grad_scale), rt.ptr(clip), rt.stream_ptr(p.device))
    rt.check(rc, "prb_adamw")
