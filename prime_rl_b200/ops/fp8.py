"""Block-scaled fp8 (e4m3) linear algebra: 1 x 128 activation scales, 128 x 128 weight scales
(``csrc/gemm_fp8.cu``; weights are quantised with ``models/fp8.py`` or in flight by the weight
push).

Training (``fp8_linear`` / ``fp8_grouped_linear``; reference: src/prime_rl/trainer/models/layers/fp8_linear.py:18-81,
layers/fp8_grouped_gemm.py:97-215): the forward product and the input gradient run on the fp8 kernel, with the
activations (and the incoming gradient) quantised per token in 1 x 128 groups along the contraction and the weight
(for the input gradient: its transpose) in 128 x 128 blocks; the weight gradient stays a bf16 product that adds into
the fp32 gradient accumulator. The fp8 copies of a weight and of its transpose are made once per optimizer step."""

from __future__ import annotations

import torch

from . import _runtime as rt


def quantize_act(x: torch.Tensor, row_valid: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """x bf16 [M, K] -> (e4m3 as uint8 [M, K], fp32 scales [M, ceil(K/128)]). ``row_valid`` (int32 [M]):
    rows with a negative entry are padding; on a GPU they are neither read nor written."""
    M, K = x.shape
    KB = (K + 127) // 128
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x if x.stride(1) == 1 else x.contiguous()
        q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
        s = torch.empty(M, KB, dtype=torch.float32, device=x.device)
        rt.check(rt.lib().prb_act_quant_fp8(x.data_ptr(), x.stride(0), q.data_ptr(), s.data_ptr(), M, K,
                                            rt.ptr(row_valid), rt.stream_ptr(x.device)), "prb_act_quant_fp8")
        return q, s
    pad = torch.zeros(M, KB * 128, dtype=torch.float32, device=x.device)
    pad[:, :K] = x.float() if row_valid is None else torch.where((row_valid >= 0)[:, None], x.float(), 0.0)
    blocks = pad.view(M, KB, 128)
    s = blocks.abs().amax(-1).clamp_min(1e-12) / 448.0
    q = (blocks / s[..., None]).view(M, KB * 128)[:, :K].to(torch.float8_e4m3fn)
    return q.view(torch.uint8), s


def fp8_gemm_ref(aq, sa, bq, sb, block_expert=None) -> torch.Tensor:
    """fp32 reference: dequantise, then multiply. bq: [N, K] or [E, N, K] (uint8 / float8)."""
    a = aq.view(torch.float8_e4m3fn).float() * sa.repeat_interleave(128, 1)[:, :aq.shape[1]]

    def deq(bq_e, sb_e):
        N, K = bq_e.shape
        s = sb_e.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
        return bq_e.view(torch.float8_e4m3fn).float() * s

    if block_expert is None:
        return a @ deq(bq, sb).t()
    out = torch.zeros(a.shape[0], bq.shape[1], dtype=torch.float32, device=a.device)
    for blk, e in enumerate(block_expert.tolist()):
        if e >= 0:
            rows = slice(blk * 128, min((blk + 1) * 128, a.shape[0]))
            out[rows] = a[rows] @ deq(bq[e], sb[e]).t()
    return out


def fp8_gemm(aq, sa, bq, sb, *, block_expert: torch.Tensor | None = None, out: torch.Tensor | None = None,
             row_valid: torch.Tensor | None = None) -> torch.Tensor:
    """C bf16 [M, N] = dequant(aq, sa) @ dequant(bq, sb)^T. Grouped when ``block_expert`` is given
    (``bq`` [E, N, K], ``sb`` [E, ceil(N/128), ceil(K/128)], rows in 128-row expert blocks).
    ``row_valid`` (int32 [M]): rows with a negative entry are padding whose inputs may be uninitialised
    and whose outputs are not stored."""
    M, K = aq.shape
    N = bq.shape[-2]
    if not aq.is_cuda:
        if row_valid is not None:           # padding rows may hold anything: keep them out of the arithmetic
            aq, sa = aq.clone(), sa.clone()
            aq[row_valid < 0] = 0
            sa[row_valid < 0] = 0
        return fp8_gemm_ref(aq, sa, bq, sb, block_expert).to(torch.bfloat16)
    assert aq.is_contiguous() and bq.is_contiguous() and sa.is_contiguous() and sb.is_contiguous()
    assert bq.shape[-1] == K and K % 16 == 0
    E = bq.shape[0] if block_expert is not None else 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    status = rt.status_tensor(aq.device)
    rt.check(rt.lib().prb_gemm_fp8(aq.data_ptr(), sa.data_ptr(), bq.data_ptr(), sb.data_ptr(), out.data_ptr(), M, N, K,
                                   out.stride(0), rt.ptr(block_expert), E, rt.ptr(row_valid), status.data_ptr(),
                                   rt.stream_ptr(aq.device)),
             "prb_gemm_fp8")
    return out


# ------------------------------------------------------------------------------------------ training
_WEIGHT_EPOCH = 0
_WEIGHT_CACHE: dict[int, tuple] = {}
CACHE_WEIGHTS = True        # False: quantise at every use (parameter sharding: a whole-model fp8 copy would undo it)
FP8_WGRAD = False           # True: the dense projections' weight gradient is an fp8 product too (quantization.wgrad)


def bump_weight_epoch() -> None:
    """Called after every optimizer step: the fp8 copies of the weights are stale."""
    global _WEIGHT_EPOCH
    _WEIGHT_EPOCH += 1
    _WEIGHT_CACHE.clear()


def _quantize_weight(w: torch.Tensor):
    from ..models.fp8 import quantize_to_fp8_blockwise

    q, s = quantize_to_fp8_blockwise(w.detach())
    return q.view(torch.uint8).contiguous(), s.contiguous()


def weight_fp8(w: torch.Tensor, transposed: bool):
    """(e4m3 as uint8, 128 x 128 scales) of ``w`` ([N, K] or [E, N, K]) or of its transpose over the last two dims."""
    key = (id(w), transposed)
    hit = _WEIGHT_CACHE.get(key) if CACHE_WEIGHTS else None
    if hit is not None and hit[0] == _WEIGHT_EPOCH and hit[1] == w.data_ptr():
        return hit[2], hit[3]
    src = w.detach().transpose(-1, -2).contiguous() if transposed else w.detach()
    q, s = _quantize_weight(src.to(torch.bfloat16) if src.is_cuda else src)
    if CACHE_WEIGHTS:
        _WEIGHT_CACHE[key] = (_WEIGHT_EPOCH, w.data_ptr(), q, s)
    return q, s


class _FP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        from .matmul import grad_accumulator

        ctx.save_for_backward(x, w)
        ctx.grad_acc = grad_accumulator(w) if w.requires_grad else None
        x2 = x.reshape(-1, x.shape[-1])
        xq, xs = quantize_act(x2)
        wq, ws = weight_fp8(w, False)
        return fp8_gemm(xq, xs, wq, ws).to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .matmul import gemm

        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            gq, gs = quantize_act(dy2)
            wtq, wts = weight_fp8(w, True)
            dx = fp8_gemm(gq, gs, wtq, wts).to(x.dtype).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            x2 = x.reshape(-1, x.shape[-1])
            if FP8_WGRAD and x2.shape[0] % 16 == 0:
                # dW = dY^T X with the tokens as the contraction: dY^T quantised per 128 tokens, X^T in 128 x 128 blocks
                gq, gs = quantize_act(dy2.t().contiguous())
                xq, xs = _quantize_weight(x2.detach().t().contiguous())
                prod = fp8_gemm(gq, gs, xq, xs)
                if ctx.grad_acc is not None:
                    ctx.grad_acc.add_(prod)
                else:
                    dw = prod.to(w.dtype)
            elif ctx.grad_acc is not None and w.shape[1] % 4 == 0:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.grad_acc, beta=1.0)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def fp8_linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w^T with the forward product and the input gradient in block-scaled fp8."""
    y = _FP8Linear.apply(x if x.is_contiguous() else x.contiguous(), w)
    return y if bias is None else y + bias.to(y.dtype)


class _FP8GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, block_expert, expert_offset):
        from .matmul import grad_accumulator

        ctx.save_for_backward(x, w, block_expert, expert_offset)
        ctx.grad_acc = grad_accumulator(w) if w.requires_grad else None
        xq, xs = quantize_act(x)
        wq, ws = weight_fp8(w, False)
        return fp8_gemm(xq, xs, wq, ws, block_expert=block_expert).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        from .matmul import grouped_wgrad

        x, w, block_expert, expert_offset = ctx.saved_tensors
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            gq, gs = quantize_act(dy)
            wtq, wts = weight_fp8(w, True)
            dx = fp8_gemm(gq, gs, wtq, wts, block_expert=block_expert).to(x.dtype)
        if ctx.needs_input_grad[1]:
            if ctx.grad_acc is not None and w.shape[2] % 4 == 0:
                grouped_wgrad(dy, x, expert_offset, w.shape[0], out=ctx.grad_acc, beta=1.0)
            else:
                dw = grouped_wgrad(dy, x, expert_offset, w.shape[0])
        return dx, dw, None, None


def fp8_grouped_linear(x, w, block_expert, expert_offset):
    """Per-expert y = x @ w[e]^T over 128-row blocks (``ops.grouped_linear``) with the forward product and the input
    gradient in block-scaled fp8."""
    return _FP8GroupedLinear.apply(x, w, block_expert, expert_offset)
