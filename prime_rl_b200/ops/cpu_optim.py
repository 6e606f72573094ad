"""Front end of the C++ CPU optimizer (``csrc/cpu/cpu_optim.cpp``), used when optimizer state
lives in host memory (``model.optim_cpu_offload`` / ``model.full_offload``)."""

from __future__ import annotations

import torch

from .. import native


def _p(t):
    return None if t is None else t.data_ptr()


def cpu_adamw_step(p, m, v, grad, out_param=None, *, step, lr, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, grad_scale=1.0):
    """In-place AdamW on contiguous CPU tensors: fp32 ``p / m / v``; ``grad`` fp32 or bf16;
    ``out_param`` (optional) receives the new parameters in bf16 or fp32."""
    assert p.device.type == "cpu" and p.dtype == torch.float32 and p.is_contiguous()
    assert grad.dtype in (torch.float32, torch.bfloat16) and grad.is_contiguous()
    if out_param is not None:
        assert out_param.dtype in (torch.float32, torch.bfloat16) and out_param.is_contiguous()
    rc = native.cpu().prb_cpu_adamw_step(p.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                                         int(grad.dtype == torch.bfloat16), _p(out_param),
                                         int(out_param is not None and out_param.dtype == torch.bfloat16), p.numel(),
                                         int(step), lr, b1, b2, eps, wd, grad_scale)
    assert rc == 0


def cpu_sign_sgd_step(p, grad, out_param=None, *, lr, wd=0.0, grad_scale=1.0):
    rc = native.cpu().prb_cpu_sign_sgd_step(p.data_ptr(), grad.data_ptr(), int(grad.dtype == torch.bfloat16),
                                            _p(out_param),
                                            int(out_param is not None and out_param.dtype == torch.bfloat16),
                                            p.numel(), lr, wd, grad_scale)
    assert rc == 0


def bf16_to_fp32_(dst, src, accumulate: bool = False):
    """dst (fp32) = src (bf16), or dst += src."""
    assert dst.dtype == torch.float32 and src.dtype == torch.bfloat16 and dst.numel() == src.numel()
    rc = native.cpu().prb_cpu_bf16_to_fp32(dst.data_ptr(), src.data_ptr(), dst.numel(), int(accumulate))
    assert rc == 0
