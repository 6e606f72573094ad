"""bf16 GEMM front end (tcgen05 kernel in ``csrc/gemm.cu``) and the autograd linear layers
built on it.

``gemm(a, b, a_mn=..., b_mn=...)`` follows the kernel's operand convention:

* ``a`` is ``[M, K]`` (K-major) or, with ``a_mn``, the stored tensor is ``[K, M]``;
* ``b`` is ``[N, K]`` (K-major, the ``nn.Linear`` weight layout) or, with ``b_mn``, ``[K, N]``.

CPU tensors (and non-bf16 dtypes) run the PyTorch reference, which is also the oracle of
the GPU tests.
"""

from __future__ import annotations

import torch

from . import _runtime as rt
from . import stash


# Dense GEMMs whose 128 x 256 output tiles cover at most half of the SMs (decode-sized projections) may split
# their reduction over several CTAs per tile (a second kernel adds the fp32 partials); the scratch for the
# partials is kept per device and stream.
SPLITK_WS_BYTES = 32 << 20
_splitk_ws: dict = {}


def _splitk_scratch(device: torch.device) -> torch.Tensor:
    key = (device.index, rt.stream_ptr(device))
    got = _splitk_ws.get(key)
    if got is None:
        got = _splitk_ws[key] = torch.empty(SPLITK_WS_BYTES, dtype=torch.uint8, device=device)
    return got


def gemm_ref(a, b, *, a_mn=False, b_mn=False, out_dtype=None, alpha=1.0, beta=0.0, out=None):
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    res = alpha * (A.float() @ B.float())
    if beta != 0.0 and out is not None:
        res = res + beta * out.float()
    res = res.to(out_dtype or a.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    block_expert: torch.Tensor | None = None,
    num_experts: int = 0,
    b_rows_per_expert: int = 0,
    n: int | None = None,
    force_bn: int = 0,
    ext: tuple[torch.Tensor, torch.Tensor] | None = None,
    row_valid: torch.Tensor | None = None,
    splitk: int = 0,
    block_ready: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> torch.Tensor:
    """C = alpha * A.B + beta * C. ``splitk``: pin the number of reduction splits of a small dense GEMM (0 = the
    kernel's cost model decides, 1 = none). Grouped mode when ``block_expert`` is given: ``b`` is the
    stacked expert weight ``[E, rows, cols]`` and ``n`` the output width. ``ext = (a2, b2)`` adds
    ``a2.b2`` in the same pass (``a2``: [M, K2]; ``b2`` laid out like ``b`` with reduction K2)."""
    if not a.is_cuda or a.dtype != torch.bfloat16:
        if block_expert is not None:
            res = grouped_gemm_ref(a, b, block_expert, b_mn=b_mn, out_dtype=torch.float32, n=n)
            if ext is not None:
                res = res + grouped_gemm_ref(ext[0], ext[1], block_expert, b_mn=b_mn, out_dtype=torch.float32, n=n)
            return res.to(out_dtype or a.dtype)
        if ext is not None:
            res = gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32) + \
                gemm_ref(ext[0], ext[1], b_mn=b_mn, out_dtype=torch.float32)
            res = alpha * res + (beta * out.float() if (beta != 0.0 and out is not None) else 0.0)
            res = res.to(out_dtype or a.dtype)
            if out is not None:
                out.copy_(res)
                return out
            return res
        return gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype, alpha=alpha, beta=beta, out=out)
    assert a.dim() == 2 and a.stride(1) == 1 and b.stride(-1) == 1
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    grouped = block_expert is not None
    if grouped:
        assert b.dim() == 3 and b.is_contiguous()
        num_experts = b.shape[0]
        b_rows_per_expert = b.shape[1]
        N = n if n is not None else (b.shape[2] if b_mn else b.shape[1])
        kb = b.shape[1] if b_mn else b.shape[2]
        ldb = b.shape[2]
    else:
        assert b.dim() == 2
        N = b.shape[1] if b_mn else b.shape[0]
        kb = b.shape[0] if b_mn else b.shape[1]
        ldb = b.stride(0)
    assert kb == K, f"reduction mismatch {kb} vs {K}"
    if not grouped and ext is None and (a.stride(0) % 8 or ldb % 8 or a.data_ptr() % 16 or b.data_ptr() % 16):
        # TMA needs 16-byte aligned bases and row pitches; odd little operands (a 4-expert router, a
        # per-head gate) are not worth a copy into padded buffers
        return gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype or (out.dtype if out is not None else None),
                        alpha=alpha, beta=beta, out=out)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        assert beta == 0.0
    assert out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    status = rt.status_tensor(a.device)
    if ext is not None:
        a2, b2 = ext
        assert not a_mn and a2.dim() == 2 and a2.shape[0] == M and a2.stride(1) == 1 and b2.stride(-1) == 1
        K2 = a2.shape[1]
        if grouped:
            assert b2.dim() == 3 and b2.is_contiguous() and b2.shape[0] == num_experts
            assert (b2.shape[1] if b_mn else b2.shape[2]) == K2
            ldb2, b2_rows = b2.shape[2], b2.shape[1]
        else:
            assert b2.dim() == 2 and (b2.shape[0] if b_mn else b2.shape[1]) == K2
            ldb2, b2_rows = b2.stride(0), 0
        rc = rt.lib().prb_gemm_bf16_ext(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), ldb, out.stride(0),
            int(a_mn), int(b_mn), int(out.dtype == torch.float32), float(alpha), float(beta),
            rt.ptr(block_expert), int(num_experts), int(b_rows_per_expert), int(force_bn),
            a2.data_ptr(), b2.data_ptr(), K2, a2.stride(0), ldb2, b2_rows,
            status.data_ptr(), rt.stream_ptr(a.device),
        )
        rt.check(rc, "prb_gemm_bf16_ext")
        return out
    if block_ready is not None:
        # grouped GEMM over rows that other GPUs are still writing: the loader waits per 128-row block until
        # arrived[b] >= expected[b]
        arrived, expected = block_ready
        assert grouped and not a_mn and ext is None and row_valid is None and alpha == 1.0 and beta == 0.0
        assert arrived.dtype == torch.int32 and expected.dtype == torch.int32 and arrived.numel() * 128 >= M
        rc = rt.lib().prb_gemm_bf16_grouped_arrive(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), ldb, out.stride(0), int(b_mn),
            int(out.dtype == torch.float32), block_expert.data_ptr(), int(num_experts), int(b_rows_per_expert),
            arrived.data_ptr(), expected.data_ptr(), status.data_ptr(), rt.stream_ptr(a.device),
        )
        rt.check(rc, "prb_gemm_bf16_grouped_arrive")
        return out
    if row_valid is not None:
        # inference-only: rows with row_valid < 0 (int32 per row of C) are not stored
        assert row_valid.dtype == torch.int32 and row_valid.numel() >= M and not a_mn
        rc = rt.lib().prb_gemm_bf16_rowmask(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), ldb, out.stride(0),
            int(a_mn), int(b_mn), int(out.dtype == torch.float32), float(alpha), float(beta),
            rt.ptr(block_expert), int(num_experts), int(b_rows_per_expert), int(force_bn),
            row_valid.data_ptr(), status.data_ptr(), rt.stream_ptr(a.device),
        )
        rt.check(rc, "prb_gemm_bf16_rowmask")
        return out
    if not grouped and not a_mn and K >= 512 and -(-M // 128) * -(-N // 256) * 2 <= rt.sm_count(a.device):
        # too few output tiles for the SMs: let the kernel split the reduction (it decides by its cost model)
        ws = _splitk_scratch(a.device)
        rc = rt.lib().prb_gemm_bf16_splitk(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), ldb, out.stride(0), int(b_mn),
            int(out.dtype == torch.float32), float(alpha), float(beta), ws.data_ptr(), ws.numel(),
            int(force_bn), int(splitk), status.data_ptr(), rt.stream_ptr(a.device),
        )
        rt.check(rc, "prb_gemm_bf16_splitk")
        return out
    rc = rt.lib().prb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), ldb, out.stride(0),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), float(alpha), float(beta),
        rt.ptr(block_expert), int(num_experts), int(b_rows_per_expert), int(force_bn),
        status.data_ptr(), rt.stream_ptr(a.device),
    )
    rt.check(rc, "prb_gemm_bf16")
    return out


def grouped_gemm_ref(a, w, block_expert, *, b_mn=False, out_dtype=None, n=None):
    """Rows of ``a`` come in 128-row blocks owned by ``block_expert[blk]`` (-1 = unused)."""
    E = w.shape[0]
    N = n if n is not None else (w.shape[2] if b_mn else w.shape[1])
    out = torch.zeros(a.shape[0], N, dtype=out_dtype or a.dtype, device=a.device)
    be = block_expert.tolist()
    for blk, e in enumerate(be):
        if e < 0 or e >= E:
            continue
        rows = slice(blk * 128, min((blk + 1) * 128, a.shape[0]))
        W = w[e].float() if b_mn else w[e].float().t()
        out[rows] = (a[rows].float() @ W).to(out.dtype)
    return out


def grad_accumulator(w: torch.Tensor):
    """fp32 tensor of ``w``'s shape into which weight gradients are to be accumulated directly (set on the
    parameter by the flat-buffer optimizer), or None: the weight-gradient GEMM then adds its product to it in
    its epilogue (``beta = 1``, fp32 output) instead of materialising a bf16 gradient that is added in a
    second pass (which reads and writes 12 bytes per parameter and micro-batch)."""
    acc = getattr(w, "_grad_acc", None)
    if acc is None or not acc.is_cuda or acc.dtype != torch.float32 or not acc.is_contiguous() or \
            acc.shape != w.shape or acc.data_ptr() % 16:
        return None
    return acc


class _Linear(torch.autograd.Function):
    """y = x @ w^T with all three GEMMs on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.grad_acc = grad_accumulator(w) if w.requires_grad else None
        x2 = x.reshape(-1, x.shape[-1])
        y = stash.run("mm", lambda: gemm(x2, w))          # selective recomputation keeps this product
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            x2 = x.reshape(-1, x.shape[-1])
            if ctx.grad_acc is not None and w.shape[1] % 4 == 0:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.grad_acc, beta=1.0)     # dw stays None: already added
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16) or \
            (stash.active() and x.dtype == w.dtype):          # the stash lives in the autograd function
        if not x.is_contiguous():
            x = x.contiguous()
        y = _Linear.apply(x, w)
    else:
        y = torch.nn.functional.linear(x, w.to(x.dtype))
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y


class _GroupedLinear(torch.autograd.Function):
    """Per-expert y = x @ w[e]^T over 128-row blocks; x is the permuted, padded row space."""

    @staticmethod
    def forward(ctx, x, w, block_expert, expert_offset, out=None, block_ready=None):
        ctx.save_for_backward(x, w, block_expert, expert_offset)
        ctx.grad_acc = grad_accumulator(w) if w.requires_grad else None
        # a caller that owns the memory of the input gradient (the peer-memory EP dispatcher)
        # hangs it on the input tensor; the backward then writes straight into it
        ctx.grad_out = getattr(x, "_grad_out_buf", None)
        if out is not None:          # the caller's buffer is shared between layers: its contents cannot be kept
            return gemm(x, w, block_expert=block_expert, out=out, block_ready=block_ready)
        if block_ready is not None:  # must run: it is the wait for rows that peers are still writing
            return gemm(x, w, block_expert=block_expert, block_ready=block_ready)
        return stash.run("grouped_mm", lambda: gemm(x, w, block_expert=block_expert))

    @staticmethod
    def backward(ctx, dy):
        x, w, block_expert, expert_offset = ctx.saved_tensors
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            go = ctx.grad_out if (ctx.grad_out is not None and ctx.grad_out.shape == x.shape) else None
            dx = gemm(dy, w, b_mn=True, block_expert=block_expert, out=go)
        if ctx.needs_input_grad[1]:
            if ctx.grad_acc is not None and w.shape[2] % 4 == 0:
                grouped_wgrad(dy, x, expert_offset, w.shape[0], out=ctx.grad_acc, beta=1.0)
            else:
                dw = grouped_wgrad(dy, x, expert_offset, w.shape[0])
        return dx, dw, None, None, None, None


def grouped_linear(x, w, block_expert, expert_offset, out=None, block_ready=None):
    return _GroupedLinear.apply(x, w, block_expert, expert_offset, out, block_ready)


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, expert_offset: torch.Tensor, num_experts: int,
                  out: torch.Tensor | None = None, beta: float = 0.0) -> torch.Tensor:
    """dW[e] = dY_e^T @ X_e over the (128-aligned) row range of each expert; with ``out`` / ``beta`` the
    product is added to an existing (fp32) accumulator."""
    E = num_experts
    N, K = dy.shape[1], x.shape[1]
    if x.is_cuda and x.dtype == torch.bfloat16:
        # one k-grouped launch over the experts' row ranges, no host read of the offsets
        from .lora import kgrouped_gemm

        return kgrouped_gemm(dy, x, expert_offset, E, out_dtype=x.dtype, out=out, beta=beta)
    assert out is None, "accumulating weight gradients in place is the GPU path"
    dw = torch.empty(E, N, K, dtype=x.dtype, device=x.device)
    offs = expert_offset.tolist()
    for e in range(E):
        r0, r1 = offs[e], offs[e + 1]
        if r1 <= r0:
            dw[e].zero_()
            continue
        if x.is_cuda and x.dtype == torch.bfloat16:
            gemm(dy[r0:r1], x[r0:r1], a_mn=True, b_mn=True, out=dw[e])
        else:
            dw[e] = (dy[r0:r1].float().t() @ x[r0:r1].float()).to(x.dtype)
    return dw
