"""Decoder building blocks. Activations are packed token-major (``[T, ...]``, one row per
token of the packed micro-batch); document structure travels in ``SeqInfo``.

Projections are stored fused (``qkv_proj``, ``gate_up_proj``) because that is how the
kernels consume them; ``models/convert.py`` maps to and from the canonical per-projection
names that checkpoints use (the reference does the same with state-dict hooks,
src/prime_rl/trainer/models/fusions.py:47-67).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import lora as lora_ops
from ..ops import moe as moe_ops
from .config import ModelArch


@dataclass
class SeqInfo:
    """Document layout of one packed micro-batch."""

    cu_seqlens: torch.Tensor      # int32 [num_docs + 1]
    max_seqlen: int
    position_ids: torch.Tensor    # int32 [T]
    # optional per-layer expert ids captured by the rollout engine ([T, layers, k])
    routed_experts: torch.Tensor | None = None
    cp: object | None = None      # context-parallel state (parallel/cp.py)
    # attention outputs kept across activation recomputation, keyed by layer (ops/attention.py)
    attn_cache: dict | None = None
    # outputs of GEMM-class operators kept across recomputation in "selective" mode (ops/stash.py)
    op_stash: object | None = None
    # values one layer leaves for later layers of the same forward (sparse-attention indices)
    shared: dict | None = None
    # rotary angles [T, rotary_dim / 2] when positions have several axes (multimodal MRoPE); attention
    # layers that support it use these instead of position_ids * inv_freq
    mrope_angles: torch.Tensor | None = None
    # rollout engine: an object that holds what precedes the new tokens (paged K / V, convolution tails, recurrent
    # states) and answers ``attend / conv / mamba / delta`` for them (engine/hybrid.py)
    engine: object | None = None

    @classmethod
    def from_lengths(cls, lengths: list[int], device) -> "SeqInfo":
        cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lengths, dtype=torch.int32).cumsum(0)
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]) if lengths else torch.zeros(0, dtype=torch.int32)
        return cls(cu.to(device), max(lengths) if lengths else 0, pos.to(device))


def _init(t: torch.Tensor, std: float) -> torch.Tensor:
    return nn.init.normal_(t, mean=0.0, std=std)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


class LoRAAdapter(nn.Module):
    """Rank-r adapter for a (possibly fused) projection: one (A, B) pair per segment.
    ``lora_A`` is stored stacked ``[S*r, in]``; ``lora_B`` per segment ``[out_s, r]``
    (``[E, ...]`` leading dim for experts)."""

    def __init__(self, in_dim: int, seg_sizes: list[int], rank: int, alpha: float, names: list[str],
                 num_experts: int | None = None, dtype=None, device=None):
        super().__init__()
        self.rank, self.scale, self.names, self.seg_sizes = rank, alpha / rank, names, seg_sizes
        lead = () if num_experts is None else (num_experts,)
        self.lora_A = nn.Parameter(torch.empty(*lead, len(seg_sizes) * rank, in_dim, dtype=dtype, device=device))
        self.lora_B = nn.ParameterList(
            [nn.Parameter(torch.zeros(*lead, s, rank, dtype=dtype, device=device)) for s in seg_sizes])
        self.reset()

    def reset(self, seed: int | None = None):
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.lora_A.device).manual_seed(seed)
        bound = 1.0 / math.sqrt(self.lora_A.shape[-1])
        with torch.no_grad():
            self.lora_A.uniform_(-bound, bound, generator=gen)
            for b in self.lora_B:
                b.zero_()


class MultiLoRA(nn.ModuleList):
    """Several adapters of one projection (one per concurrent run); which one a token uses follows from
    ``set_lora_num_tokens`` (reference: src/prime_rl/trainer/models/layers/lora/base.py:14-60,
    multi_linear.py:38)."""

    def ops_args(self):
        return [(a.lora_A, list(a.lora_B), a.scale) for a in self]


_LORA_NUM_TOKENS: list[torch.Tensor | None] = [None]


def set_lora_num_tokens(num_tokens: torch.Tensor | None) -> None:
    """``num_tokens[i]`` consecutive tokens of the coming forward pass use adapter i (a micro-batch is sorted by
    adapter). ``None``: every token uses adapter 0."""
    _LORA_NUM_TOKENS[0] = num_tokens


def get_lora_num_tokens(total: int, device) -> torch.Tensor:
    t = _LORA_NUM_TOKENS[0]
    if t is None:
        return torch.tensor([total], dtype=torch.int32, device=device)
    return t.to(device)


class Linear(nn.Module):
    """Bias-free (by default) projection ``[out, in]`` with an optional LoRA adapter."""

    def __init__(self, in_dim: int, out_dim: int, bias: bool = False, std: float = 0.02, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_dim, in_dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_dim, dtype=dtype, device=device)) if bias else None
        self.lora: LoRAAdapter | None = None
        self.std = std
        self.fp8: tuple[torch.Tensor, torch.Tensor] | None = None    # (e4m3 weight, 128 x 128 scales): inference only
        self.fp8_train = False      # forward product and input gradient in block-scaled fp8 (model.quantization)

    def reset_parameters(self):
        _init(self.weight, self.std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def quantize_fp8_(self, drop_bf16: bool = False, source: torch.Tensor | None = None) -> bool:
        """(Re)builds the block-scaled fp8 copy of the weight used by no-grad forwards. ``source``: new
        bf16 values to quantise instead of ``self.weight`` (a weight update of a module whose bf16 copy
        was dropped). ``drop_bf16``: afterwards release the bf16 storage; the module then serves from
        the fp8 copy only (serving engines: the freed memory goes to the KV cache)."""
        w = source if source is not None else self.weight.data
        if self.lora is not None or w.numel() == 0 or w.shape[1] % 16 or not w.is_cuda:
            return False
        from .fp8 import quantize_to_fp8_blockwise

        q, s = quantize_to_fp8_blockwise(w.to(torch.bfloat16))
        if self.fp8 is None:
            self.fp8 = (q.view(torch.uint8).contiguous(), s.contiguous())
        else:                           # keep the buffers (a peer-memory weight push may write into them)
            self.fp8[0].copy_(q.view(torch.uint8))
            self.fp8[1].copy_(s)
        if drop_bf16:
            self.fp8_shape = tuple(w.shape)
            self.weight.data = torch.empty(0, dtype=self.weight.dtype, device=self.weight.device)
        return True

    def forward(self, x):
        if self.fp8 is not None and not torch.is_grad_enabled() and x.dtype == torch.bfloat16:
            from ..ops import fp8 as fp8_ops

            x2 = x.reshape(-1, x.shape[-1])
            xq, xs = fp8_ops.quantize_act(x2)
            y = fp8_ops.fp8_gemm(xq, xs, self.fp8[0], self.fp8[1]).reshape(*x.shape[:-1], self.fp8[0].shape[0])
            return y if self.bias is None else y + self.bias
        if isinstance(self.lora, MultiLoRA):
            nt = get_lora_num_tokens(x.numel() // x.shape[-1], x.device)
            y = lora_ops.multi_lora_linear(x, self.weight, self.lora.ops_args(), nt)
            return y if self.bias is None else y + self.bias
        if self.lora is not None:
            y = lora_ops.lora_linear(x, self.weight, self.lora.lora_A, list(self.lora.lora_B), self.lora.scale)
            return y if self.bias is None else y + self.bias
        if self.fp8_train and torch.is_grad_enabled() and x.dtype == self.weight.dtype:
            from ..ops import fp8 as fp8_ops

            return fp8_ops.fp8_linear(x, self.weight, self.bias)
        return ops.linear(x, self.weight, self.bias)


class Attention(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, attn_backend: str = "auto", dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx, self.backend = arch, layer_idx, attn_backend
        H, D = arch.hidden_size, arch.head_dim
        self.nq, self.nkv, self.D = arch.layer_heads(layer_idx), arch.num_key_value_heads, D
        q_dim = self.nq * D
        std = arch.initializer_range
        self.qkv_proj = Linear(H, q_dim + 2 * arch.kv_dim, bias=arch.attention_bias, std=std, dtype=dtype,
                               device=device)
        self.o_proj = Linear(q_dim, H, bias=arch.attention_bias and arch.model_type == "gpt_oss", std=std,
                             dtype=dtype, device=device)
        # softplus output gate computed from the layer input: one value per head or per channel
        # (reference: LagunaFlashAttention, src/prime_rl/trainer/models/laguna/modeling_laguna.py:101-165)
        self.g_proj = None
        if arch.attn_gate != "none":
            self.g_proj = Linear(H, self.nq if arch.attn_gate == "per_head" else q_dim, std=std, dtype=dtype,
                                 device=device)
        if arch.qk_norm:
            self.q_norm = RMSNorm(D, arch.rms_norm_eps, dtype=dtype, device=device)
            self.k_norm = RMSNorm(D, arch.rms_norm_eps, dtype=dtype, device=device)
        else:
            self.q_norm = self.k_norm = None
        self.sinks = nn.Parameter(torch.zeros(self.nq, dtype=dtype, device=device)) if arch.attention_sinks else None
        self.window = arch.layer_window(layer_idx)
        inv_f = ops.inv_freq(D, arch.rope_theta, device=device, rotary_dim=arch.rotary_dim)
        if not arch.use_rope:
            inv_f = torch.zeros_like(inv_f)         # angle 0 everywhere: the rotation is the identity
        self.register_buffer("inv_freq", inv_f, persistent=False)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        T = x.shape[0]
        qkv = self.qkv_proj(x)
        q_dim, kv_dim = self.nq * self.D, self.nkv * self.D
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        q, k, v = ops.qkv_norm_rope(qkv, qw, kw, seq.position_ids, self.inv_freq, self.arch.rms_norm_eps, self.nq,
                                    self.nkv, self.D)
        if seq.engine is not None:
            o = seq.engine.attend(self.layer_idx, q, k, v, self.window, self.sinks)
        elif seq.cp is not None:
            o = seq.cp.attention(q, k, v, seq, window=self.window, sinks=self.sinks, backend=self.backend)
        else:
            o = attn_ops.attention(q, k, v, seq.cu_seqlens, seq.max_seqlen, causal=True, window=self.window,
                                   sinks=self.sinks, backend=self.backend, cache=seq.attn_cache,
                                   cache_key=self.layer_idx)
        return self.finish(o, x)

    def finish(self, o: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """Output gate (when the family has one) and output projection; ``x`` is the layer input."""
        T = o.shape[0]
        if self.g_proj is not None:
            gate = torch.nn.functional.softplus(self.g_proj(x).float()).to(o.dtype)
            o = o * (gate.unsqueeze(-1) if self.arch.attn_gate == "per_head" else gate.view(T, self.nq, self.D))
        return self.o_proj(o.reshape(T, self.nq * self.D))


_ACT = {"silu": act_ops.SWIGLU, "swiglu_clamped": act_ops.SWIGLU_CLAMPED, "relu2": act_ops.RELU2,
        "silu_clamped": act_ops.SILU_CLAMPED}


class DenseMLP(nn.Module):
    def __init__(self, arch: ModelArch, intermediate: int | None = None, dtype=None, device=None):
        super().__init__()
        I = intermediate or arch.intermediate_size
        self.act = _ACT[arch.hidden_act]
        self.arch = arch
        width = I if self.act == act_ops.RELU2 else 2 * I
        self.gate_up_proj = Linear(arch.hidden_size, width, std=arch.initializer_range, dtype=dtype, device=device)
        self.down_proj = Linear(I, arch.hidden_size, std=arch.initializer_range, dtype=dtype, device=device)

    def forward(self, x):
        gu = self.gate_up_proj(x)
        return self.down_proj(ops.glu(gu, self.act, self.arch.swiglu_limit, self.arch.swiglu_alpha))


class Router(nn.Module):
    """Token-choice top-k router: gate projection (fp32 accumulate and output), softmax or
    sigmoid scores, optional selection bias, optional replay of engine-chosen experts
    (reference: TokenChoiceTopKRouter, src/prime_rl/trainer/models/layers/moe.py:182-322)."""

    def __init__(self, arch: ModelArch, dtype=None, device=None):
        super().__init__()
        self.arch = arch
        self.gate = Linear(arch.hidden_size, arch.num_experts, bias=arch.router_linear_bias,
                           std=arch.initializer_range, dtype=dtype, device=device)
        if arch.router_bias:
            self.register_buffer("e_score_correction_bias", torch.zeros(arch.num_experts, dtype=torch.float32,
                                                                        device=device))
        else:
            self.e_score_correction_bias = None
        self.force_balanced = False
        self.want_plan = False            # set by the owning MoE layer when it runs its experts locally
        self.last_plan = None             # the experts' row plan, when the last forward built it with the selection

    def forward(self, x: torch.Tensor, forced: torch.Tensor | None = None):
        a = self.arch
        if x.is_cuda and x.dtype == torch.bfloat16:
            logits = _RouterLogits.apply(x, self.gate.weight)
        else:
            logits = (x.float() @ self.gate.weight.float().t())
        if self.gate.bias is not None:
            logits = logits + self.gate.bias.float()
        if self.force_balanced and forced is None:
            T = x.shape[0]
            base = torch.arange(T, device=x.device)[:, None] * a.num_experts_per_tok
            forced = ((base + torch.arange(a.num_experts_per_tok, device=x.device)[None, :]) % a.num_experts)
        self.last_plan = None
        if self.want_plan:
            # decode-sized inference batches: selection, histogram and the row plan of the experts in one launch
            fused = moe_ops.route_and_plan_small(logits, a.num_experts_per_tok, score_func=a.score_func,
                                                 norm_topk=a.norm_topk_prob, route_scale=a.routed_scaling_factor,
                                                 sel_bias=self.e_score_correction_bias, forced=forced)
            if fused is not None:
                idx, w, counts, self.last_plan = fused
                return idx, w, counts, logits
        idx, w, counts = moe_ops.route_topk(logits, a.num_experts_per_tok, score_func=a.score_func,
                                            norm_topk=a.norm_topk_prob, route_scale=a.routed_scaling_factor,
                                            sel_bias=self.e_score_correction_bias, forced=forced)
        return idx, w, counts, logits


class _RouterLogits(torch.autograd.Function):
    """bf16 operands, fp32 accumulate, fp32 logits (the reference's moe_router_dtype=float32)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return ops.gemm(x, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dlogits):
        x, w = ctx.saved_tensors
        dl = dlogits.to(torch.bfloat16)
        dx = ops.gemm(dl, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = ops.gemm(dl, x, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw


class GroupedExperts(nn.Module):
    """Stacked expert weights ``gate_up_proj [E, 2I, H]`` and ``down_proj [E, H, I]``."""

    def __init__(self, arch: ModelArch, num_local_experts: int | None = None, dtype=None, device=None):
        super().__init__()
        self.arch = arch
        E = num_local_experts or arch.num_experts
        I, H = arch.moe_intermediate_size, arch.expert_hidden
        self.act = _ACT[arch.hidden_act]
        width = I if self.act == act_ops.RELU2 else 2 * I
        self.gate_up_proj = nn.Parameter(torch.empty(E, width, H, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(E, H, I, dtype=dtype, device=device))
        # per-expert projection biases (GPT-OSS): [gate | up] in the row order of gate_up_proj
        self.gate_up_proj_bias = nn.Parameter(torch.zeros(E, width, dtype=dtype, device=device)) if arch.expert_bias else None
        self.down_proj_bias = nn.Parameter(torch.zeros(E, H, dtype=dtype, device=device)) if arch.expert_bias else None
        self.lora_gate_up: LoRAAdapter | None = None
        self.lora_down: LoRAAdapter | None = None
        self.fp8: dict[str, tuple[torch.Tensor, torch.Tensor]] | None = None   # inference-only fp8 copies
        self.fp8_train = False      # both projections' forward products and input gradients in block-scaled fp8

    def reset_parameters(self):
        _init(self.gate_up_proj, self.arch.initializer_range)
        _init(self.down_proj, self.arch.initializer_range)

    def quantize_fp8_(self, drop_bf16: bool = False, source: dict[str, torch.Tensor] | None = None) -> bool:
        """Block-scaled fp8 copies of both expert stacks (see ``Linear.quantize_fp8_``); ``source`` maps
        ``gate_up_proj`` / ``down_proj`` to new bf16 values."""
        if self.lora_gate_up is not None or self.lora_down is not None:
            return False
        from .fp8 import quantize_to_fp8_blockwise

        done = False
        for name in ("gate_up_proj", "down_proj"):
            p = getattr(self, name)
            w = source.get(name) if source is not None else p.data
            if w is None or w.numel() == 0 or not w.is_cuda:
                continue
            if self.fp8 is None:
                self.fp8 = {}
            # expert by expert: the fp32 staging of the quantiser never exceeds one expert
            q, s = quantize_to_fp8_blockwise(w.to(torch.bfloat16))
            if name not in self.fp8:
                self.fp8[name] = (q.view(torch.uint8).contiguous(), s.contiguous())
            else:
                self.fp8[name][0].copy_(q.view(torch.uint8))
                self.fp8[name][1].copy_(s)
            if drop_bf16:
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            done = True
        return done

    def _biased(self, y: torch.Tensor, bias: torch.Tensor | None, block_expert: torch.Tensor) -> torch.Tensor:
        """Adds every row's expert bias (rows come in 128-row blocks owned by ``block_expert``; unused blocks
        borrow expert 0, nothing reads them)."""
        if bias is None:
            return y
        row_expert = block_expert.clamp_min(0).long().repeat_interleave(128)[:y.shape[0]]
        return y + bias[row_expert].to(y.dtype)

    def supports_fp8_row_mask(self, x: torch.Tensor) -> bool:
        """No-grad forward from the fp8 copies on the GPU: the token rows are quantised once, gathered as
        fp8 into the expert-sorted order, and the padding rows are skipped by every kernel."""
        return (not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16 and self.fp8 is not None
                and self.gate_up_proj_bias is None
                and self.act != act_ops.SILU_CLAMPED and x.shape[1] % 512 == 0)

    def forward_fp8_masked(self, x: torch.Tensor, plan) -> torch.Tensor:
        """``x`` [T, H] bf16 (unpermuted) -> expert outputs [P, H] in the plan's row order; rows with
        ``plan.row_src < 0`` are left unwritten."""
        from ..ops import fp8 as fp8_ops
        from ..ops import moe as moe_ops

        T, H = x.shape
        xq, xs = fp8_ops.quantize_act(x)                              # T rows, not T * k
        # the fp8 payload and its scales travel through the row gather as opaque 16-bit words
        xpq = moe_ops.permute_nopad(xq.view(torch.bfloat16), plan).view(torch.uint8)
        xps = moe_ops.permute_nopad(xs.view(torch.bfloat16), plan).view(torch.float32)
        valid = plan.row_src
        gu = fp8_ops.fp8_gemm(xpq, xps, *self.fp8["gate_up_proj"], block_expert=plan.block_expert, row_valid=valid)
        h = act_ops.glu_rowmask(gu, valid, self.act, self.arch.swiglu_limit, self.arch.swiglu_alpha)
        hq, hs = fp8_ops.quantize_act(h, row_valid=valid)
        return fp8_ops.fp8_gemm(hq, hs, *self.fp8["down_proj"], block_expert=plan.block_expert, row_valid=valid)

    def supports_row_mask(self, x: torch.Tensor) -> bool:
        """No-grad bf16 forward on the GPU without adapters or fp8 copies: the padding rows that round every
        expert up to 128 need not be written, read by the activation or stored by the GEMMs."""
        return (not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16 and self.fp8 is None
                and self.gate_up_proj_bias is None
                and self.lora_gate_up is None and self.lora_down is None and self.act != act_ops.SILU_CLAMPED
                and self.gate_up_proj.dtype == torch.bfloat16)

    def supports_block_ready(self, x: torch.Tensor) -> bool:
        """The first projection is the plain bf16 grouped GEMM, whose loader can wait per 128-row block for rows
        that other GPUs are still writing (``forward(block_ready=...)``)."""
        return (x.is_cuda and x.dtype == torch.bfloat16 and self.lora_gate_up is None
                and self.gate_up_proj.dtype == torch.bfloat16
                and not (self.fp8 is not None and not torch.is_grad_enabled()))

    def forward(self, xp: torch.Tensor, block_expert: torch.Tensor, expert_offset: torch.Tensor,
                out: torch.Tensor | None = None, row_valid: torch.Tensor | None = None,
                block_ready: tuple[torch.Tensor, torch.Tensor] | None = None,
                row_adapter: torch.Tensor | None = None) -> torch.Tensor:
        """``out`` (optional, ``[P, H]`` bf16): memory the last projection writes into. ``row_valid``
        (int32 per permuted row, < 0 = padding; only where ``supports_row_mask``): those rows are skipped.
        ``block_ready = (arrived, expected)`` (only where ``supports_block_ready``): per 128-row block of ``xp``,
        a counter that its writers raise and the row count at which the block is complete."""
        assert block_ready is None or (row_valid is None and self.supports_block_ready(xp))
        if row_valid is not None:
            gu = ops.gemm(xp, self.gate_up_proj, block_expert=block_expert, row_valid=row_valid)
            h = act_ops.glu_rowmask(gu, row_valid, self.act, self.arch.swiglu_limit, self.arch.swiglu_alpha)
            return ops.gemm(h, self.down_proj, block_expert=block_expert, out=out, row_valid=row_valid)
        if self.fp8 is not None and not torch.is_grad_enabled() and xp.dtype == torch.bfloat16:
            from ..ops import fp8 as fp8_ops

            xq, xs = fp8_ops.quantize_act(xp)
            gu = fp8_ops.fp8_gemm(xq, xs, *self.fp8["gate_up_proj"], block_expert=block_expert)
            gu = self._biased(gu, self.gate_up_proj_bias, block_expert)
            h = ops.glu(gu, self.act, self.arch.swiglu_limit, self.arch.swiglu_alpha)
            hq, hs = fp8_ops.quantize_act(h)
            if self.down_proj_bias is not None:
                return self._biased(fp8_ops.fp8_gemm(hq, hs, *self.fp8["down_proj"], block_expert=block_expert),
                                    self.down_proj_bias, block_expert)
            return fp8_ops.fp8_gemm(hq, hs, *self.fp8["down_proj"], block_expert=block_expert, out=out)
        if isinstance(self.lora_gate_up, MultiLoRA):
            if row_adapter is None:
                raise ValueError("several adapters on the experts need the adapter of every permuted row")
            gu = lora_ops.multi_lora_grouped_linear(xp, self.gate_up_proj, self.lora_gate_up.ops_args(), row_adapter,
                                                    block_expert, expert_offset)
        elif self.lora_gate_up is not None:
            l = self.lora_gate_up
            gu = lora_ops.lora_grouped_linear(xp, self.gate_up_proj, l.lora_A, list(l.lora_B), l.scale, block_expert,
                                              expert_offset)
        elif self.fp8_train and torch.is_grad_enabled() and block_ready is None:
            from ..ops import fp8 as fp8_ops

            gu = fp8_ops.fp8_grouped_linear(xp, self.gate_up_proj, block_expert, expert_offset)
        else:
            gu = ops.grouped_linear(xp, self.gate_up_proj, block_expert, expert_offset, block_ready=block_ready)
        gu = self._biased(gu, self.gate_up_proj_bias, block_expert)
        h = ops.glu(gu, self.act, self.arch.swiglu_limit, self.arch.swiglu_alpha)
        if self.down_proj_bias is not None:
            out = None                # the bias add makes a new tensor anyway
        if isinstance(self.lora_down, MultiLoRA):
            y = lora_ops.multi_lora_grouped_linear(h, self.down_proj, self.lora_down.ops_args(), row_adapter,
                                                   block_expert, expert_offset, out=out)
        elif self.lora_down is not None:
            l = self.lora_down
            y = lora_ops.lora_grouped_linear(h, self.down_proj, l.lora_A, list(l.lora_B), l.scale, block_expert,
                                             expert_offset, out=out)
        elif self.fp8_train and torch.is_grad_enabled() and out is None:
            from ..ops import fp8 as fp8_ops

            y = fp8_ops.fp8_grouped_linear(h, self.down_proj, block_expert, expert_offset)
        else:
            y = ops.grouped_linear(h, self.down_proj, block_expert, expert_offset, out=out)
        return self._biased(y, self.down_proj_bias, block_expert)


class MoE(nn.Module):
    """Router -> dispatch (local permute, or expert-parallel all-to-all) -> grouped experts
    -> combine, plus optional shared experts."""

    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx = arch, layer_idx
        self.router = Router(arch, dtype=dtype, device=device)
        self.experts = GroupedExperts(arch, dtype=dtype, device=device)
        if arch.n_shared_experts > 0:
            self.shared_experts = DenseMLP(arch, arch.shared_width, dtype=dtype,
                                           device=device)
        else:
            self.shared_experts = None
        self.shared_expert_gate = None
        if arch.shared_expert_gate and self.shared_experts is not None:
            self.shared_expert_gate = Linear(arch.hidden_size, 1, std=arch.initializer_range, dtype=dtype, device=device)
        # experts that work in a projected ("latent") space: project in before dispatch, out after combine
        self.fc1_latent_proj = self.fc2_latent_proj = None
        if arch.moe_latent_size:
            self.fc1_latent_proj = Linear(arch.hidden_size, arch.moe_latent_size, std=arch.initializer_range,
                                          dtype=dtype, device=device)
            self.fc2_latent_proj = Linear(arch.moe_latent_size, arch.hidden_size, std=arch.initializer_range,
                                          dtype=dtype, device=device)
        self.dispatcher = None            # parallel/ep.py installs an expert-parallel dispatcher here
        # (lo, hi): this process holds only those experts while every token is present on every rank (the serving
        # engine's expert parallelism, engine/tp.py); the output is then a partial sum that the caller reduces
        self.expert_range: tuple[int, int] | None = None
        self.last_counts: torch.Tensor | None = None
        self.last_topk: torch.Tensor | None = None     # [T, k] expert ids of the last forward (router replay capture)
        self.last_router_stats: dict | None = None

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        T = x.shape[0]
        forced = None
        if seq.routed_experts is not None:
            forced = seq.routed_experts[:, self.layer_idx, :].to(torch.int32)
        self.router.want_plan = self.dispatcher is None and self.expert_range is None
        idx, w, counts, logits = self.router(x, forced)
        self.last_counts = counts
        self.last_topk = idx
        xe = x if self.fc1_latent_proj is None else self.fc1_latent_proj(x)
        if self.dispatcher is not None:
            if isinstance(self.experts.lora_gate_up, MultiLoRA):
                raise NotImplementedError("several adapters on expert-parallel experts: the adapter ids of the "
                                          "dispatched rows are not exchanged")
            y = self.dispatcher(self.experts, xe, idx, w, counts)
        else:
            plan = self.router.last_plan
            if plan is None:
                plan = moe_ops.build_plan(idx, counts, self.arch.num_experts, expert_range=self.expert_range)
            if self.experts.supports_fp8_row_mask(xe):
                yp = self.experts.forward_fp8_masked(xe, plan)
            elif self.experts.supports_row_mask(xe) and xe.shape[1] % 8 == 0:
                # inference: nothing touches the rows that only pad every expert to a multiple of 128
                xp = moe_ops.permute_nopad(xe, plan)
                yp = self.experts(xp, plan.block_expert, plan.expert_offset, row_valid=plan.row_src)
            elif isinstance(self.experts.lora_gate_up, MultiLoRA):
                # adapter of the token that every permuted row came from (-1: padding row)
                tok_adapter = lora_ops.adapter_of_token(get_lora_num_tokens(T, x.device), T)
                src = plan.row_src.long()
                row_adapter = torch.where(src >= 0, tok_adapter[src.clamp(min=0) // plan.k], -1)
                xp = moe_ops.permute(xe, plan)
                yp = self.experts(xp, plan.block_expert, plan.expert_offset, row_adapter=row_adapter)
            else:
                xp = moe_ops.permute(xe, plan)
                yp = self.experts(xp, plan.block_expert, plan.expert_offset)
            y = moe_ops.combine(yp, w, plan, T)
        if self.fc2_latent_proj is not None:
            y = self.fc2_latent_proj(y)
        if self.shared_experts is not None:
            sh = self.shared_experts(x)
            if self.shared_expert_gate is not None:
                sh = sh * torch.sigmoid(self.shared_expert_gate(x).float()).to(sh.dtype)
            y = y + sh
        return y


def _token_mixer(arch: ModelArch, layer_idx: int, attn_backend: str, dtype, device) -> nn.Module:
    kind = arch.mixer_type(layer_idx)
    if kind == "attention":
        return Attention(arch, layer_idx, attn_backend, dtype=dtype, device=device)
    from . import mixers

    if kind == "gated_attention":
        return mixers.GatedAttention(arch, layer_idx, attn_backend, dtype=dtype, device=device)
    if kind == "gated_delta_net":
        return mixers.GatedDeltaNet(arch, layer_idx, dtype=dtype, device=device)
    if kind == "mla_dsa":
        return mixers.SparseMLAAttention(arch, layer_idx, dtype=dtype, device=device)
    raise ValueError(f"unknown token mixer '{kind}'")


class SingleMixerBlock(nn.Module):
    """One pre-normed mixer per layer, ``h + mixer(norm(h))``: the Nemotron-H layout, where a
    layer is a Mamba-2 mixer, an attention, a dense MLP or an MoE
    (reference: NemotronHDecoderLayer, src/prime_rl/trainer/models/nemotron_h/modeling_nemotron_h.py:45-125)."""

    def __init__(self, arch: ModelArch, layer_idx: int, attn_backend: str = "auto", dtype=None, device=None):
        super().__init__()
        self.kind = arch.block_type(layer_idx)
        self.norm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)
        self.is_moe = self.kind == "moe"
        if self.kind == "mamba":
            from . import mixers

            self.mamba = mixers.Mamba2Mixer(arch, layer_idx, dtype=dtype, device=device)
        elif self.kind == "attention":
            self.self_attn = Attention(arch, layer_idx, attn_backend, dtype=dtype, device=device)
        elif self.kind == "moe":
            self.mlp = MoE(arch, layer_idx, dtype=dtype, device=device)
        elif self.kind == "mlp":
            self.mlp = DenseMLP(arch, dtype=dtype, device=device)
        else:
            raise ValueError(f"unknown block type '{self.kind}'")

    def forward(self, h: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        x = self.norm(h)
        if self.kind == "mamba":
            return h + self.mamba(x, seq)
        if self.kind == "attention":
            return h + self.self_attn(x, seq)
        return h + (self.mlp(x, seq) if self.is_moe else self.mlp(x))


class DecoderLayer(nn.Module):
    def __new__(cls, arch: ModelArch, layer_idx: int, *args, **kwargs):
        if cls is DecoderLayer and arch.block_types is not None:
            return SingleMixerBlock(arch, layer_idx, *args, **kwargs)
        return super().__new__(cls)

    def __init__(self, arch: ModelArch, layer_idx: int, attn_backend: str = "auto", dtype=None, device=None):
        super().__init__()
        self.input_layernorm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)
        self.self_attn = _token_mixer(arch, layer_idx, attn_backend, dtype, device)
        self.post_attention_layernorm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)
        if arch.layer_is_moe(layer_idx):
            self.mlp = MoE(arch, layer_idx, dtype=dtype, device=device)
        else:
            self.mlp = DenseMLP(arch, dtype=dtype, device=device)
        self.is_moe = arch.layer_is_moe(layer_idx)

    def forward(self, h: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        a = self.self_attn(self.input_layernorm(h), seq)
        x, h = ops.add_rms_norm(a, h, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        m = self.mlp(x, seq) if self.is_moe else self.mlp(x)
        return h + m
