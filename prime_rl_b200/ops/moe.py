"""MoE routing / permutation front end (``csrc/moe.cu``) — no host synchronisation: every
shape is a static upper bound and the data-dependent sizes live on the device.

``RoutingPlan`` describes where each (token, choice) pair sits in the expert-sorted row
space in which every expert's rows start on a 128-row boundary.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _runtime as rt


@dataclass
class RoutingPlan:
    topk_idx: torch.Tensor       # [T, k] int32
    slot: torch.Tensor           # [T, k] int32 row of each pair in the permuted space
    row_src: torch.Tensor        # [P] int32: t*k + j, or -1 for padding
    expert_offset: torch.Tensor  # [E+1] int32, 128-aligned starts
    block_expert: torch.Tensor   # [P/128] int32, -1 past the used rows
    total_rows: torch.Tensor     # [1] int32
    counts: torch.Tensor         # [E] int32 tokens per expert
    max_rows: int                # P
    k: int
    num_experts: int


def max_padded_rows(num_pairs: int, num_experts: int) -> int:
    """Static upper bound of the padded row count: each expert wastes at most 127 rows."""
    return (num_pairs + num_experts * 127 + 127) // 128 * 128


def router_scores_ref(logits, score_func="softmax"):
    return torch.softmax(logits.float(), dim=-1) if score_func == "softmax" else torch.sigmoid(logits.float())


def route_topk(logits: torch.Tensor, k: int, *, score_func: str = "softmax", norm_topk: bool = True,
               route_scale: float = 1.0, sel_bias: torch.Tensor | None = None,
               forced: torch.Tensor | None = None):
    """Returns (topk_idx [T,k] int32, topk_w [T,k] fp32 differentiable w.r.t. logits, counts [E])."""
    T, E = logits.shape
    if logits.is_cuda and logits.dtype == torch.float32 and E <= 1024:
        # selection, weights and histogram in one kernel (no host synchronisation, unlike
        # bincount); when gradients are needed the weights are rebuilt differentiably from the
        # kernel's choice
        idx32, w_nd, counts, _ = router_topk_cuda(logits.detach().contiguous(), k, score_func=score_func,
                                                  norm_topk=norm_topk, route_scale=route_scale, sel_bias=sel_bias,
                                                  forced=None if forced is None else forced.to(torch.int32).contiguous())
        if not (torch.is_grad_enabled() and logits.requires_grad):
            return idx32, w_nd, counts
        w = router_scores_ref(logits, score_func).gather(1, idx32.long())
        if norm_topk:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return idx32, w * route_scale, counts
    scores = router_scores_ref(logits, score_func)
    if forced is not None:
        idx = forced.long()
    else:
        sel = scores if sel_bias is None else scores + sel_bias.float()
        idx = torch.topk(sel.detach(), k, dim=-1).indices
    w = scores.gather(1, idx)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * route_scale
    counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
    return idx.to(torch.int32), w, counts


# Tokens up to which one CTA routes and plans in a single launch: one token per warp of the 1024-thread CTA.
# Beyond that the single SM is the bottleneck (measured: 256 tokens cost 85 us against 20 us for the separate
# kernels), so larger batches keep the multi-CTA router followed by the plan and scatter kernels.
SMALL_ROUTE_TOKENS = 32


def route_and_plan_small(logits: torch.Tensor, k: int, *, score_func: str = "softmax", norm_topk: bool = True,
                         route_scale: float = 1.0, sel_bias: torch.Tensor | None = None,
                         forced: torch.Tensor | None = None):
    """Inference-only, small decode batches (``T <= SMALL_ROUTE_TOKENS``): ``route_topk`` and
    ``build_plan`` in ONE kernel launch. Returns (topk_idx, topk_w, counts, plan), or None where the
    kernel does not apply (the caller then uses the separate ops)."""
    T, E = logits.shape
    if (not logits.is_cuda or logits.dtype != torch.float32 or E > 512 or k > 16 or T == 0 or T > SMALL_ROUTE_TOKENS
            or T * k > 8192 or torch.is_grad_enabled()):
        return None
    dev = logits.device
    logits = logits.contiguous()
    P = max_padded_rows(T * k, E)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    w = torch.empty(T, k, dtype=torch.float32, device=dev)
    # counts [E] | expert_offset [E + 1] | total [1] | block_expert [P / 128] | slot [T k] | row_src [P] in one allocation
    sizes = [E, E + 1, 1, P // 128, T * k, P]
    buf = torch.empty(sum(sizes), dtype=torch.int32, device=dev)
    counts, expert_offset, total, block_expert, slot, row_src = buf.split(sizes)
    forced32 = None if forced is None else forced.to(torch.int32).contiguous()
    rc = rt.lib().prb_moe_route_plan_small(logits.data_ptr(), rt.ptr(sel_bias), rt.ptr(forced32), idx.data_ptr(),
                                           w.data_ptr(), None, counts.data_ptr(), expert_offset.data_ptr(),
                                           block_expert.data_ptr(), total.data_ptr(), slot.data_ptr(), row_src.data_ptr(),
                                           T, E, k, P // 128, 0 if score_func == "softmax" else 1, int(norm_topk),
                                           float(route_scale), rt.stream_ptr(dev))
    rt.check(rc, "prb_moe_route_plan_small")
    plan = RoutingPlan(idx, slot.view(T, k), row_src, expert_offset, block_expert, total, counts, P, k, E)
    return idx, w, counts, plan


def build_plan(topk_idx: torch.Tensor, counts: torch.Tensor, num_experts: int, deterministic: bool = False,
               expert_range: tuple[int, int] | None = None) -> RoutingPlan:
    """``expert_range = (lo, hi)``: this rank owns only those experts of the ``num_experts`` (tokens replicated, experts
    split: the serving engine's expert parallelism). The plan then covers ``hi - lo`` local experts; pairs of other
    experts get ``slot = -1`` and no row, and ``combine`` leaves their term to the rank that owns them."""
    T, k = topk_idx.shape
    E = num_experts
    if expert_range is not None:
        return _build_plan_range(topk_idx, counts, expert_range, deterministic)
    P = max_padded_rows(T * k, E)
    dev = topk_idx.device
    if topk_idx.is_cuda:
        if topk_idx.dtype != torch.int32 or counts.dtype != torch.int32 or not topk_idx.is_contiguous():
            raise TypeError("build_plan on a GPU takes contiguous int32 expert ids and int32 counts")
        expert_offset = torch.empty(E + 1, dtype=torch.int32, device=dev)
        block_expert = torch.empty(P // 128, dtype=torch.int32, device=dev)
        cursor = torch.empty(E, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        slot = torch.empty(T, k, dtype=torch.int32, device=dev)
        row_src = torch.empty(P, dtype=torch.int32, device=dev)
        rc = rt.lib().prb_moe_plan(topk_idx.data_ptr(), counts.data_ptr(), expert_offset.data_ptr(),
                                   block_expert.data_ptr(), cursor.data_ptr(), total.data_ptr(), slot.data_ptr(),
                                   row_src.data_ptr(), T, E, k, P // 128, int(deterministic), rt.stream_ptr(dev))
        rt.check(rc, "prb_moe_plan")
        return RoutingPlan(topk_idx, slot, row_src, expert_offset, block_expert, total, counts, P, k, E)
    # CPU reference: stable order inside each expert
    flat = topk_idx.reshape(-1).long()
    padded = (counts.long() + 127) // 128 * 128
    expert_offset = torch.zeros(E + 1, dtype=torch.long)
    expert_offset[1:] = padded.cumsum(0)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    starts = torch.zeros(E, dtype=torch.long)
    starts[1:] = counts.long().cumsum(0)[:-1]
    rank_in_e = torch.arange(flat.numel()) - starts[sorted_e]
    pos = expert_offset[sorted_e] + rank_in_e
    slot = torch.empty(flat.numel(), dtype=torch.long)
    slot[order] = pos
    row_src = torch.full((P,), -1, dtype=torch.int32)
    row_src[pos] = order.to(torch.int32)
    blk_rows = torch.arange(P // 128) * 128
    block_expert = torch.searchsorted(expert_offset[1:].contiguous(), blk_rows, right=True).to(torch.int32)
    block_expert[blk_rows >= expert_offset[E]] = -1
    return RoutingPlan(topk_idx, slot.reshape(T, k).to(torch.int32), row_src, expert_offset.to(torch.int32),
                       block_expert, expert_offset[E:].to(torch.int32), counts, P, k, E)


def _build_plan_range(topk_idx, counts, expert_range, deterministic) -> RoutingPlan:
    lo, hi = expert_range
    T, k = topk_idx.shape
    E = hi - lo
    P = max_padded_rows(T * k, E)
    dev = topk_idx.device
    local_counts = counts[lo:hi].contiguous()
    if topk_idx.is_cuda:
        expert_offset = torch.empty(E + 1, dtype=torch.int32, device=dev)
        block_expert = torch.empty(P // 128, dtype=torch.int32, device=dev)
        cursor = torch.empty(E, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        slot = torch.empty(T, k, dtype=torch.int32, device=dev)
        row_src = torch.empty(P, dtype=torch.int32, device=dev)
        rc = rt.lib().prb_moe_plan_range(topk_idx.data_ptr(), local_counts.data_ptr(), expert_offset.data_ptr(),
                                         block_expert.data_ptr(), cursor.data_ptr(), total.data_ptr(), slot.data_ptr(),
                                         row_src.data_ptr(), T, E, k, P // 128, int(deterministic), lo,
                                         rt.stream_ptr(dev))
        rt.check(rc, "prb_moe_plan_range")
        return RoutingPlan(topk_idx, slot, row_src, expert_offset, block_expert, total, local_counts, P, k, E)
    flat = topk_idx.reshape(-1).long() - lo
    mine = (flat >= 0) & (flat < E)
    pairs = torch.nonzero(mine).reshape(-1)                       # pair ids (t * k + j) of the owned experts
    padded = (local_counts.long() + 127) // 128 * 128
    expert_offset = torch.zeros(E + 1, dtype=torch.long)
    expert_offset[1:] = padded.cumsum(0)
    order = pairs[torch.argsort(flat[pairs], stable=True)]
    sorted_e = flat[order]
    starts = torch.zeros(E, dtype=torch.long)
    starts[1:] = local_counts.long().cumsum(0)[:-1]
    pos = expert_offset[sorted_e] + torch.arange(order.numel()) - starts[sorted_e]
    slot = torch.full((flat.numel(),), -1, dtype=torch.long)
    slot[order] = pos
    row_src = torch.full((P,), -1, dtype=torch.int32)
    row_src[pos] = order.to(torch.int32)
    blk_rows = torch.arange(P // 128) * 128
    block_expert = torch.searchsorted(expert_offset[1:].contiguous(), blk_rows, right=True).to(torch.int32)
    block_expert[blk_rows >= expert_offset[E]] = -1
    return RoutingPlan(topk_idx, slot.reshape(T, k).to(torch.int32), row_src, expert_offset.to(torch.int32),
                       block_expert, expert_offset[E:].to(torch.int32), local_counts, P, k, E)


class _Permute(torch.autograd.Function):
    """x [T, H] -> permuted rows [P, H] (padding rows zero)."""

    @staticmethod
    def forward(ctx, x, plan: RoutingPlan):
        ctx.plan = plan
        ctx.T = x.shape[0]
        return _gather_rows(x, plan, None)

    @staticmethod
    def backward(ctx, dp):
        plan = ctx.plan
        return _combine(dp.contiguous(), plan, None, None, ctx.T), None


class _Combine(torch.autograd.Function):
    """y[t] = sum_j w[t, j] * p[slot[t, j]]."""

    @staticmethod
    def forward(ctx, p, w, plan: RoutingPlan, T):
        ctx.plan = plan
        ctx.save_for_backward(p, w)
        return _combine(p, plan, w, None, T)

    @staticmethod
    def backward(ctx, dy):
        p, w = ctx.saved_tensors
        plan = ctx.plan
        dy = dy.contiguous()
        dp = _gather_rows(dy, plan, w.detach().reshape(-1).contiguous()) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            T, k = plan.slot.shape
            if dy.is_cuda:
                dw = torch.empty(T, k, dtype=torch.float32, device=dy.device)
                rc = rt.lib().prb_moe_combine_bwd_w(dy.data_ptr(), p.data_ptr(), plan.slot.data_ptr(), dw.data_ptr(),
                                                    T, dy.shape[1], k, rt.stream_ptr(dy.device))
                rt.check(rc, "prb_moe_combine_bwd_w")
            else:
                dw = (p[plan.slot.long()].float() * dy.float()[:, None, :]).sum(-1)
        return dp, dw, None, None


def _gather_rows(x, plan: RoutingPlan, w, zero_pad: bool = True):
    P, H = plan.max_rows, x.shape[1]
    if x.is_cuda and x.dtype == torch.bfloat16 and H % 8 == 0:
        out = torch.empty(P, H, dtype=x.dtype, device=x.device)
        fn = rt.lib().prb_moe_gather_rows if zero_pad else rt.lib().prb_moe_gather_rows_nopad
        rc = fn(x.data_ptr(), plan.row_src.data_ptr(), rt.ptr(w), out.data_ptr(), P, H,
                plan.k, plan.total_rows.data_ptr(), rt.stream_ptr(x.device))
        rt.check(rc, "prb_moe_gather_rows")
        return out
    src = plan.row_src.long()
    valid = src >= 0
    out = torch.zeros(P, H, dtype=x.dtype, device=x.device)
    rows = x[(src[valid] // plan.k)]
    if w is not None:
        rows = (rows.float() * w[src[valid]].float()[:, None]).to(x.dtype)
    out[valid] = rows
    return out


def _combine(p, plan: RoutingPlan, w, residual, T):
    H = p.shape[1]
    if p.is_cuda and p.dtype == torch.bfloat16 and H % 8 == 0:
        y = torch.empty(T, H, dtype=p.dtype, device=p.device)
        wf = w.detach().float().contiguous() if w is not None else None
        rc = rt.lib().prb_moe_combine(p.data_ptr(), plan.slot.data_ptr(), rt.ptr(wf), rt.ptr(residual), y.data_ptr(),
                                      T, H, plan.k, rt.stream_ptr(p.device))
        rt.check(rc, "prb_moe_combine")
        return y
    sl = plan.slot.long()
    rows = p[sl.clamp(min=0)].float() * (sl >= 0)[..., None]  # [T, k, H]; slot < 0: the pair belongs to another rank
    if w is not None:
        rows = rows * w.float()[:, :, None]
    y = rows.sum(1)
    if residual is not None:
        y = y + residual.float()
    return y.to(p.dtype)


def permute(x: torch.Tensor, plan: RoutingPlan) -> torch.Tensor:
    return _Permute.apply(x, plan)


def permute_nopad(x: torch.Tensor, plan: RoutingPlan) -> torch.Tensor:
    """Inference-only ``permute``: the padding rows (``plan.row_src < 0``) are left uninitialised; the grouped
    GEMMs / GLU that follow must be given ``row_valid=plan.row_src`` so that they skip those rows."""
    return _gather_rows(x, plan, None, zero_pad=False)


def combine(p: torch.Tensor, w: torch.Tensor, plan: RoutingPlan, num_tokens: int) -> torch.Tensor:
    return _Combine.apply(p, w, plan, num_tokens)


def router_topk_cuda(logits: torch.Tensor, k: int, *, score_func="softmax", norm_topk=True, route_scale=1.0,
                     sel_bias=None, forced=None):
    """Fused scores + top-k + histogram; returns (idx, weights, counts, scores). Not
    differentiable: callers rebuild the weights from ``scores`` when they need gradients."""
    T, E = logits.shape
    dev = logits.device
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    w = torch.empty(T, k, dtype=torch.float32, device=dev)
    scores = torch.empty(T, E, dtype=torch.float32, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    rc = rt.lib().prb_router_topk(logits.data_ptr(), rt.ptr(sel_bias), rt.ptr(forced), idx.data_ptr(), w.data_ptr(),
                                  scores.data_ptr(), counts.data_ptr(), T, E, k,
                                  0 if score_func == "softmax" else 1, int(norm_topk), float(route_scale),
                                  rt.stream_ptr(dev))
    rt.check(rc, "prb_router_topk")
    return idx, w, counts, scores
