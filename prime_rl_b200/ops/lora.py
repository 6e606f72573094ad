"""LoRA-adapted linear layers with the adapter GEMMs fused into the base projection's output.

``lora_linear``          y = x W^T + scale * sum_s (x A_s^T) B_s^T written into the column
                         segment of s (a fused qkv / gate_up projection has one adapter per
                         original projection, as the reference's per-module LoRA has);
``lora_grouped_linear``  the same per expert over the permuted 128-row-block row space
                         (the reference's MultiLoRAGroupedExperts,
                         src/prime_rl/trainer/models/layers/lora/).

The base weight is frozen (no weight gradient is formed); every product runs on the
tcgen05 GEMM. The adapter term is not a separate pass over the output: the S adapters' B
matrices are laid out block-diagonally as one ``[out, S*r]`` operand and the base GEMM takes
``(x A^T, B_blockdiag)`` as one extra reduction block into the same TMEM accumulator (TMA
zero-fills the rank-r operands up to the 64-wide block), in forward and for the input gradient.
"""

from __future__ import annotations

import torch

from .matmul import gemm, grouped_gemm_ref
from . import _runtime as rt


def _segments(seg_sizes):
    out, c = [], 0
    for s in seg_sizes:
        out.append((c, c + s))
        c += s
    return out


def lora_linear_ref(x, w, a_cat, b_list, scale):
    """Differentiable PyTorch reference. a_cat: [S*r, in]; b_list[s]: [out_s, r]."""
    r = b_list[0].shape[1]
    y = x @ w.to(x.dtype).t()
    t = x @ a_cat.to(x.dtype).t()
    parts = [t[..., s * r:(s + 1) * r] @ b.to(x.dtype).t() for s, b in enumerate(b_list)]
    return y + scale * torch.cat(parts, dim=-1)


def _block_diag(b_list, scale, rows=None):
    """[.., out_s, r] x S -> [.., out, S*r] with B_s * scale in its own r columns. ``rows[s] = (c0, c1)`` places
    block s at output rows c0..c1 (several adapters of one projection share rows); default: one after another."""
    r = b_list[0].shape[-1]
    S = len(b_list)
    if rows is None:
        rows = _segments([b.shape[-2] for b in b_list])
    out = max(c1 for _, c1 in rows)
    bd = torch.zeros(*b_list[0].shape[:-2], out, S * r, dtype=b_list[0].dtype, device=b_list[0].device)
    for s, b in enumerate(b_list):
        c0, c1 = rows[s]
        bd[..., c0:c1, s * r:(s + 1) * r] = b if scale == 1.0 else b * scale
    return bd


class _LoRALinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, a_cat, scale, rank_mask, rows, *b_list):
        """``rank_mask`` ([T, S*r] or None) multiplies x A^T: several adapters share one launch, every token keeps
        only the rank columns of its own adapter (times that adapter's scale)."""
        t = gemm(x, a_cat)
        if rank_mask is not None:
            t = t * rank_mask
        bd = _block_diag(b_list, scale, rows)
        y = gemm(x, w, ext=(t, bd))
        ctx.save_for_backward(x, w, a_cat, t, bd, rank_mask)
        ctx.scale = scale
        ctx.rows = rows if rows is not None else _segments([b.shape[0] for b in b_list])
        ctx.b_dtype = b_list[0].dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, a_cat, t, bd, rank_mask = ctx.saved_tensors
        scale = ctx.scale
        S = len(ctx.rows)
        r = bd.shape[1] // S
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dt = gemm(dy, bd, b_mn=True)                       # [T, S*r], scale is inside bd
        if rank_mask is not None:
            dt = dt * rank_mask
        db = []
        for s, (c0, c1) in enumerate(ctx.rows):
            db.append(gemm(dy[:, c0:c1], t[:, s * r:(s + 1) * r], a_mn=True, b_mn=True, out_dtype=torch.float32,
                           alpha=scale).to(ctx.b_dtype))
        da = gemm(dt, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(a_cat.dtype)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, b_mn=True, ext=(dt, a_cat))
        return (dx, None, da, None, None, None, *db)


def lora_linear(x, w, a_cat, b_list, scale: float):
    """x: [..., in]; w: [out, in] frozen; a_cat: [S*r, in]; b_list: S tensors [out_s, r]."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = _LoRALinear.apply(x2, w, a_cat, float(scale), None, None, *b_list)
        return y.reshape(*shape[:-1], w.shape[0])
    return lora_linear_ref(x, w, a_cat, list(b_list), scale)


def adapter_of_token(num_tokens: torch.Tensor, total: int) -> torch.Tensor:
    """``num_tokens[i]`` consecutive tokens belong to adapter i -> adapter index per token ([total] int64); no
    host read (tokens past the sum, if any, get the last adapter)."""
    ends = num_tokens.to(torch.int64).cumsum(0)
    pos = torch.arange(total, device=num_tokens.device)
    return torch.searchsorted(ends, pos, right=True).clamp_(max=num_tokens.numel() - 1)


def rank_mask_for(adapter_idx: torch.Tensor, scales, cols_per_adapter: int, dtype) -> torch.Tensor:
    """[rows, n * cols_per_adapter]: scale_i in the columns of row's adapter i, zero elsewhere."""
    n = len(scales)
    sc = torch.as_tensor(scales, dtype=torch.float32, device=adapter_idx.device)
    onehot = torch.nn.functional.one_hot(adapter_idx.clamp(min=0), n).to(torch.float32) * sc
    onehot = onehot * (adapter_idx >= 0).unsqueeze(-1)
    return onehot.repeat_interleave(cols_per_adapter, dim=1).to(dtype)


def multi_lora_linear(x, w, adapters, num_tokens: torch.Tensor):
    """Several adapters in one micro-batch (the reference's MultiLoRALinear,
    src/prime_rl/trainer/models/layers/lora/multi_linear.py:38-164): ``num_tokens[i]`` consecutive tokens use
    adapter i. ``adapters[i] = (a_cat_i [S*r, in], b_list_i (S tensors [out_s, r]), scale_i)``.

    y[t] = x[t] W^T + scale_i * sum_s (x[t] A_{i,s}^T) B_{i,s}^T for the adapter i of token t. All adapters ride in
    ONE extra reduction segment of the base GEMM: the A matrices are stacked along the rank, x A^T is masked so that
    a token keeps only its adapter's columns, and the B matrices of all adapters sit side by side over the same
    output rows."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    T = x2.shape[0]
    n = len(adapters)
    S = len(adapters[0][1])
    r = adapters[0][1][0].shape[-1]
    idx = adapter_of_token(num_tokens.to(x.device), T)
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        y = x2 @ w.to(x.dtype).t()
        add = torch.zeros_like(y)
        for i, (a_cat, b_list, scale) in enumerate(adapters):
            t = x2 @ a_cat.to(x.dtype).t()
            parts = [t[:, s * r:(s + 1) * r] @ b.to(x.dtype).t() for s, b in enumerate(b_list)]
            add = add + (idx == i).unsqueeze(-1).to(x.dtype) * (scale * torch.cat(parts, dim=-1))
        return (y + add).reshape(*shape[:-1], w.shape[0])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    a_all = torch.cat([a for a, _, _ in adapters], dim=0)                     # [n*S*r, in]
    b_all = [b for _, bl, _ in adapters for b in bl]
    seg = _segments([b.shape[0] for b in adapters[0][1]])
    mask = rank_mask_for(idx, [sc for _, _, sc in adapters], S * r, x.dtype)
    y = _LoRALinear.apply(x2, w, a_all, 1.0, mask, seg * n, *b_all)
    return y.reshape(*shape[:-1], w.shape[0])


def kgrouped_gemm(a: torch.Tensor, b: torch.Tensor, expert_offset: torch.Tensor, num_experts: int, *,
                  alpha: float = 1.0, out_dtype=torch.float32, out: torch.Tensor | None = None,
                  beta: float = 0.0) -> torch.Tensor:
    """out[e] = alpha * a_e^T @ b_e (+ beta * out[e]) over expert e's rows; a: [P, M], b: [P, N] -> [E, M, N].
    ``out`` (contiguous, bf16 or fp32) lets a weight gradient accumulate where it is kept."""
    M, N = a.shape[1], b.shape[1]
    if a.is_cuda and a.dtype == torch.bfloat16:
        if out is None:
            assert beta == 0.0
            out = torch.empty(num_experts, M, N, dtype=out_dtype, device=a.device)
        assert out.is_contiguous() and out.shape == (num_experts, M, N)
        status = rt.status_tensor(a.device)
        rc = rt.lib().prb_gemm_bf16_kgrouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, a.shape[0],
                                             a.stride(0), b.stride(0), N, int(out.dtype == torch.float32),
                                             float(alpha), float(beta), expert_offset.data_ptr(), num_experts,
                                             status.data_ptr(), rt.stream_ptr(a.device))
        rt.check(rc, "prb_gemm_bf16_kgrouped")
        return out
    offs = expert_offset.tolist()
    out = torch.zeros(num_experts, M, N, dtype=out_dtype, device=a.device)
    for e in range(num_experts):
        r0, r1 = offs[e], offs[e + 1]
        if r1 > r0:
            out[e] = (alpha * (a[r0:r1].float().t() @ b[r0:r1].float())).to(out_dtype)
    return out


def lora_grouped_linear_ref(x, w, a_cat, b_list, scale, block_expert):
    r = b_list[0].shape[2]
    y = grouped_gemm_ref(x, w, block_expert, out_dtype=torch.float32)
    t = grouped_gemm_ref(x, a_cat, block_expert, out_dtype=torch.float32)
    parts = [grouped_gemm_ref(t[:, s * r:(s + 1) * r].contiguous(), b, block_expert, out_dtype=torch.float32)
             for s, b in enumerate(b_list)]
    return (y + scale * torch.cat(parts, dim=-1)).to(x.dtype)


class _LoRAGroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, a_cat, scale, block_expert, expert_offset, out, rank_mask, rows, *b_list):
        t = gemm(x, a_cat, block_expert=block_expert)
        if rank_mask is not None:                          # several adapters: see _LoRALinear
            t = t * rank_mask
        bd = _block_diag(b_list, scale, rows)              # [E, out, S*r]
        y = gemm(x, w, block_expert=block_expert, ext=(t, bd), out=out)
        ctx.grad_out = getattr(x, "_grad_out_buf", None)   # see ops/matmul.py _GroupedLinear
        ctx.save_for_backward(x, w, a_cat, t, block_expert, expert_offset, bd, rank_mask)
        ctx.scale = scale
        ctx.rows = rows if rows is not None else _segments([b.shape[1] for b in b_list])
        ctx.b_dtype = b_list[0].dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, a_cat, t, block_expert, expert_offset, bd, rank_mask = ctx.saved_tensors
        scale = ctx.scale
        E = w.shape[0]
        S = len(ctx.rows)
        r = bd.shape[2] // S
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dt = gemm(dy, bd, b_mn=True, block_expert=block_expert)     # [P, S*r], scale is inside bd
        if rank_mask is not None:
            dt = dt * rank_mask
        db = []
        for s, (c0, c1) in enumerate(ctx.rows):
            db.append(kgrouped_gemm(dy[:, c0:c1], t[:, s * r:(s + 1) * r], expert_offset, E, alpha=scale)
                      .to(ctx.b_dtype))
        da = kgrouped_gemm(dt, x, expert_offset, E).to(a_cat.dtype)
        dx = None
        if ctx.needs_input_grad[0]:
            go = ctx.grad_out if (ctx.grad_out is not None and ctx.grad_out.shape == x.shape) else None
            dx = gemm(dy, w, b_mn=True, block_expert=block_expert, ext=(dt, a_cat), out=go)
        return (dx, None, da, None, None, None, None, None, None, *db)


def multi_lora_grouped_linear(x, w, adapters, row_adapter: torch.Tensor, block_expert, expert_offset, out=None):
    """Per-expert projection with several adapters in one micro-batch (the reference's multi-LoRA experts,
    src/prime_rl/trainer/models/layers/lora/multi_moe.py). ``row_adapter`` [P] int64: adapter of the token each
    permuted row came from (-1 for padding rows). ``adapters[i] = (a_cat_i [E, S*r, in], b_list_i, scale_i)``."""
    n = len(adapters)
    S = len(adapters[0][1])
    r = adapters[0][1][0].shape[-1]
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        from .matmul import grouped_linear

        y = grouped_linear(x, w, block_expert, expert_offset)
        for i, (a_cat, b_list, scale) in enumerate(adapters):
            t = grouped_linear(x, a_cat, block_expert, expert_offset)
            parts = [grouped_linear(t[:, s * r:(s + 1) * r].contiguous(), b, block_expert, expert_offset)
                     for s, b in enumerate(b_list)]
            y = y + (row_adapter == i).unsqueeze(-1).to(x.dtype) * (scale * torch.cat(parts, dim=-1))
        return y
    a_all = torch.cat([a for a, _, _ in adapters], dim=1)                     # [E, n*S*r, in]
    b_all = [b for _, bl, _ in adapters for b in bl]
    seg = _segments([b.shape[1] for b in adapters[0][1]])
    mask = rank_mask_for(row_adapter, [sc for _, _, sc in adapters], S * r, x.dtype)
    return _LoRAGroupedLinear.apply(x, w, a_all, 1.0, block_expert, expert_offset, out, mask, seg * n, *b_all)


def lora_grouped_linear(x, w, a_cat, b_list, scale: float, block_expert, expert_offset, out=None):
    """x: [P, in] permuted rows; w: [E, out, in] frozen; a_cat: [E, S*r, in]; b_list[s]: [E, out_s, r]."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _LoRAGroupedLinear.apply(x, w, a_cat, float(scale), block_expert, expert_offset, out, None, None,
                                        *b_list)
    # CPU: differentiable composition
    from .matmul import grouped_linear

    r = b_list[0].shape[2]
    y = grouped_linear(x, w, block_expert, expert_offset)
    t = grouped_linear(x, a_cat, block_expert, expert_offset)
    parts = [grouped_linear(t[:, s * r:(s + 1) * r].contiguous(), b, block_expert, expert_offset)
             for s, b in enumerate(b_list)]
    return y + scale * torch.cat(parts, dim=-1)
