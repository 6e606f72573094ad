"""Token mixers beyond plain softmax attention: Mamba-2 (Nemotron-H), gated delta-net and
gated softmax attention (Qwen3.5), multi-head-latent attention with the DSA sparse indexer
(GLM-MoE-DSA). All of them work on packed ``[T, hidden]`` activations with ``SeqInfo``.

Parameter names follow the reference's modules so that checkpoints map one to one:
``NemotronHMamba2`` (src/prime_rl/trainer/models/nemotron_h/mamba.py:78-236),
``Qwen3_5GatedDeltaNet`` (qwen3_5/gated_delta_net.py:19-110), ``Qwen3_5Attention``
(qwen3_5/attention.py:10-84), ``GlmMoeDsaAttention`` + ``Indexer``
(glm_moe_dsa/sparse_mla_attention.py:47-238).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import attention as attn_ops
from ..ops import delta_rule, sparse_mla, ssm
from .config import ModelArch
from .layers import Linear, RMSNorm, SeqInfo


def doc_windows(seq: SeqInfo) -> tuple[torch.Tensor, torch.Tensor]:
    """Per token: index of its document's first token and its own index + 1 (the causal window
    ``[ks, ke)`` of the sparse indexer)."""
    T = seq.position_ids.shape[0]
    me = torch.arange(T, device=seq.position_ids.device, dtype=torch.int32)
    return (me - seq.position_ids.to(torch.int32)), me + 1


class Mamba2Mixer(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx = arch, layer_idx
        self.nh, self.hd, self.ng, self.ns = arch.mamba_num_heads, arch.mamba_head_dim, arch.ssm_n_groups, arch.ssm_state_size
        self.inner = self.nh * self.hd
        self.conv_dim = self.inner + 2 * self.ng * self.ns
        std = arch.initializer_range
        self.in_proj = Linear(arch.hidden_size, self.inner + self.conv_dim + self.nh, bias=arch.mamba_proj_bias, std=std,
                              dtype=dtype, device=device)
        self.conv1d_weight = nn.Parameter(torch.empty(self.conv_dim, arch.conv_kernel, dtype=dtype, device=device))
        self.conv1d_bias = nn.Parameter(torch.zeros(self.conv_dim, dtype=dtype, device=device)) if arch.use_conv_bias else None
        self.dt_bias = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32, device=device))
        self.A_log = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32, device=device))
        self.D = nn.Parameter(torch.ones(self.nh, dtype=torch.float32, device=device))
        self.norm_weight = nn.Parameter(torch.ones(self.inner, dtype=dtype, device=device))
        self.out_proj = Linear(self.inner, arch.hidden_size, bias=arch.mamba_proj_bias, std=std, dtype=dtype, device=device)
        self.reset_ssm_parameters()

    @torch.no_grad()
    def reset_ssm_parameters(self, seed: int = 0):
        """A = -(1..heads); dt_bias = inverse softplus of log-uniform time steps in [1e-3, 1e-1]."""
        gen = torch.Generator().manual_seed(seed)
        self.A_log.copy_(torch.log(torch.arange(1, self.nh + 1, dtype=torch.float32)))
        lo, hi = math.log(1e-3), math.log(1e-1)
        ts = torch.exp(torch.rand(self.nh, generator=gen) * (hi - lo) + lo).clamp(min=1e-4)
        self.dt_bias.copy_(ts + torch.log(-torch.expm1(-ts)))
        self.D.fill_(1.0)
        nn.init.uniform_(self.conv1d_weight, -0.5, 0.5)

    def _forward_cp(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        """Context parallelism: the local tokens' projections are exchanged for the whole sequence of ``heads / cp``
        heads (B / C groups are gathered whole), convolution and scan run on those, the result goes back."""
        cp = seq.cp
        if self.nh % cp.cp:
            raise ValueError(f"{self.nh} Mamba heads cannot be split over cp = {cp.cp}")
        nh_l = self.nh // cp.cp
        h0 = cp.rank * nh_l
        gate, conv_in, dt = self.in_proj(x).split([self.inner, self.conv_dim, self.nh], dim=-1)
        hs_in, bc_in = conv_in.split([self.inner, 2 * self.ng * self.ns], dim=-1)
        hs_in = cp.seq_to_heads(hs_in.contiguous())                       # [T, nh_l * hd]
        bc_in = cp.gather_seq(bc_in)                                      # [T, 2 ng ns]
        dt = cp.seq_to_heads(dt.contiguous())                             # [T, nh_l]
        T = hs_in.shape[0]
        ch = slice(h0 * self.hd, (h0 + nh_l) * self.hd)
        w = torch.cat([self.conv1d_weight[ch], self.conv1d_weight[self.inner:]], 0)
        b = None if self.conv1d_bias is None else torch.cat([self.conv1d_bias[ch], self.conv1d_bias[self.inner:]], 0)
        pos = cp.full_positions(seq)
        conv = ssm.causal_conv1d(torch.cat([hs_in, bc_in], -1), w, b, pos, "silu")
        hs, Bm, Cm = conv.split([nh_l * self.hd, self.ng * self.ns, self.ng * self.ns], dim=-1)
        dtp = F.softplus(dt.float() + self.dt_bias[h0:h0 + nh_l])
        lo, hi = self.arch.time_step_limit
        if lo > 0.0 or math.isfinite(hi):
            dtp = dtp.clamp(lo, hi)
        # the heads of one group are consecutive: the local heads see the groups they belong to
        rep = self.nh // self.ng
        groups = torch.arange(h0, h0 + nh_l, device=x.device) // rep
        Bh = Bm.reshape(T, self.ng, self.ns)[:, groups]                   # one "group" per local head
        Ch = Cm.reshape(T, self.ng, self.ns)[:, groups]
        y = ssm.mamba2_scan(hs.reshape(T, nh_l, self.hd), dtp, -torch.exp(self.A_log.float()[h0:h0 + nh_l]), Bh, Ch,
                            self.D[h0:h0 + nh_l], pos, chunk=self.arch.ssm_chunk_size)
        y = cp.heads_to_seq(y.reshape(T, nh_l * self.hd).to(x.dtype))     # [Tl, inner]
        y = ssm.gated_rms_norm(y, gate, self.norm_weight, self.arch.rms_norm_eps, self.inner // self.ng, "silu",
                               gate_first=True)
        return self.out_proj(y)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        if seq.cp is not None and seq.engine is None:
            return self._forward_cp(x, seq)
        T = x.shape[0]
        gate, conv_in, dt = self.in_proj(x).split([self.inner, self.conv_dim, self.nh], dim=-1)
        eng = seq.engine                 # rollout engine: state of the sequences before these tokens (engine/hybrid.py)
        if eng is not None:
            conv = eng.conv(self.layer_idx, conv_in, self.conv1d_weight, self.conv1d_bias, "silu")
        else:
            conv = ssm.causal_conv1d(conv_in, self.conv1d_weight, self.conv1d_bias, seq.position_ids, "silu")
        hs, Bm, Cm = conv.split([self.inner, self.ng * self.ns, self.ng * self.ns], dim=-1)
        dtp = F.softplus(dt.float() + self.dt_bias)
        lo, hi = self.arch.time_step_limit
        if lo > 0.0 or math.isfinite(hi):
            dtp = dtp.clamp(lo, hi)
        if eng is not None:
            y = eng.mamba(self.layer_idx, hs.reshape(T, self.nh, self.hd), dtp, -torch.exp(self.A_log.float()),
                          Bm.reshape(T, self.ng, self.ns), Cm.reshape(T, self.ng, self.ns), self.D,
                          self.arch.ssm_chunk_size)
        else:
            y = ssm.mamba2_scan(hs.reshape(T, self.nh, self.hd), dtp, -torch.exp(self.A_log.float()),
                                Bm.reshape(T, self.ng, self.ns), Cm.reshape(T, self.ng, self.ns), self.D,
                                seq.position_ids, chunk=self.arch.ssm_chunk_size)
        y = ssm.gated_rms_norm(y.reshape(T, self.inner).to(x.dtype), gate, self.norm_weight, self.arch.rms_norm_eps,
                               self.inner // self.ng, "silu", gate_first=True)
        return self.out_proj(y)


class GatedDeltaNet(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx = arch, layer_idx
        self.nv, self.nk = arch.linear_num_value_heads, arch.linear_num_key_heads
        self.dk, self.dv = arch.linear_key_head_dim, arch.linear_value_head_dim
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        conv_dim = 2 * self.key_dim + self.value_dim
        H, std = arch.hidden_size, arch.initializer_range
        self.in_proj_qkv = Linear(H, conv_dim, std=std, dtype=dtype, device=device)
        self.in_proj_z = Linear(H, self.value_dim, std=std, dtype=dtype, device=device)
        self.in_proj_b = Linear(H, self.nv, std=std, dtype=dtype, device=device)
        self.in_proj_a = Linear(H, self.nv, std=std, dtype=dtype, device=device)
        self.conv1d_weight = nn.Parameter(torch.empty(conv_dim, arch.linear_conv_kernel_dim, dtype=dtype, device=device))
        self.dt_bias = nn.Parameter(torch.ones(self.nv, dtype=torch.float32, device=device))
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32, device=device))
        self.norm_weight = nn.Parameter(torch.ones(self.dv, dtype=dtype, device=device))
        self.out_proj = Linear(self.value_dim, H, std=std, dtype=dtype, device=device)
        self.reset_ssm_parameters()

    @torch.no_grad()
    def reset_ssm_parameters(self, seed: int = 0):
        gen = torch.Generator().manual_seed(seed)
        self.A_log.copy_(torch.log(torch.rand(self.nv, generator=gen) * 16 + 1e-3))
        self.dt_bias.fill_(1.0)
        nn.init.uniform_(self.conv1d_weight, -0.5, 0.5)

    def _forward_cp(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        """Context parallelism: whole sequence of ``heads / cp`` key and value heads per rank (see ``Mamba2Mixer``)."""
        cp = seq.cp
        if self.nk % cp.cp or self.nv % cp.cp:
            raise ValueError(f"{self.nk} key / {self.nv} value heads cannot be split over cp = {cp.cp}")
        nk_l, nv_l = self.nk // cp.cp, self.nv // cp.cp
        k0, v0 = cp.rank * nk_l, cp.rank * nv_l
        q_in, k_in, v_in = self.in_proj_qkv(x).split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q_in, k_in, v_in = (cp.seq_to_heads(t.contiguous()) for t in (q_in, k_in, v_in))
        T = q_in.shape[0]
        kq, kv_ = slice(k0 * self.dk, (k0 + nk_l) * self.dk), slice(v0 * self.dv, (v0 + nv_l) * self.dv)
        w = self.conv1d_weight
        wl = torch.cat([w[: self.key_dim][kq], w[self.key_dim: 2 * self.key_dim][kq], w[2 * self.key_dim:][kv_]], 0)
        pos = cp.full_positions(seq)
        qkv = ssm.causal_conv1d(torch.cat([q_in, k_in, v_in], -1), wl, None, pos, "silu")
        q, k, v = qkv.split([nk_l * self.dk, nk_l * self.dk, nv_l * self.dv], dim=-1)
        beta = torch.sigmoid(cp.seq_to_heads(self.in_proj_b(x).contiguous()).float())
        a = cp.seq_to_heads(self.in_proj_a(x).contiguous()).float()
        g = -torch.exp(self.A_log.float()[v0:v0 + nv_l]) * F.softplus(a + self.dt_bias[v0:v0 + nv_l])
        q, k = q.reshape(T, nk_l, self.dk), k.reshape(T, nk_l, self.dk)
        rep = self.nv // self.nk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        o = delta_rule.gated_delta_rule(q, k, v.reshape(T, nv_l, self.dv), g, beta, pos)
        o = cp.heads_to_seq(o.reshape(T, nv_l * self.dv).to(x.dtype))      # [Tl, value_dim]
        Tl = x.shape[0]
        z = self.in_proj_z(x).reshape(Tl, self.nv, self.dv)
        o = ssm.gated_rms_norm(o.reshape(Tl, self.nv, self.dv), z, self.norm_weight, self.arch.rms_norm_eps, self.dv,
                               "silu", gate_first=False)
        return self.out_proj(o.reshape(Tl, self.value_dim))

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        if seq.cp is not None and seq.engine is None:
            return self._forward_cp(x, seq)
        T = x.shape[0]
        eng = seq.engine                 # rollout engine: state of the sequences before these tokens (engine/hybrid.py)
        if eng is not None:
            qkv = eng.conv(self.layer_idx, self.in_proj_qkv(x), self.conv1d_weight, None, "silu")
        else:
            qkv = ssm.causal_conv1d(self.in_proj_qkv(x), self.conv1d_weight, None, seq.position_ids, "silu")
        z = self.in_proj_z(x).reshape(T, self.nv, self.dv)
        beta = torch.sigmoid(self.in_proj_b(x).float())
        g = -torch.exp(self.A_log.float()) * F.softplus(self.in_proj_a(x).float() + self.dt_bias)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k = q.reshape(T, self.nk, self.dk), k.reshape(T, self.nk, self.dk)
        rep = self.nv // self.nk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        if eng is not None:
            o = eng.delta(self.layer_idx, q, k, v.reshape(T, self.nv, self.dv), g, beta)
        else:
            o = delta_rule.gated_delta_rule(q, k, v.reshape(T, self.nv, self.dv), g, beta, seq.position_ids)
        o = ssm.gated_rms_norm(o.to(x.dtype), z, self.norm_weight, self.arch.rms_norm_eps, self.dv, "silu",
                               gate_first=False)
        return self.out_proj(o.reshape(T, self.value_dim))


def norm_rope_with_angles(x: torch.Tensor, w: torch.Tensor | None, ang: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the head dim, then the half-split rotation of the first ``2 * ang.shape[1]``
    channels by the given angles ``[T, rd / 2]`` (positions with several axes)."""
    xf = x.float()
    if w is not None:
        xf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype).float()
    rd = ang.shape[1] * 2
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2, rest = xf[..., : rd // 2], xf[..., rd // 2: rd], xf[..., rd:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest], dim=-1).to(x.dtype)


class GatedAttention(nn.Module):
    """Softmax attention whose query projection also emits a sigmoid output gate (per head:
    ``[q | gate]``), with q/k RMSNorm and partial rotary embedding."""

    def __init__(self, arch: ModelArch, layer_idx: int, attn_backend: str = "auto", dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx, self.backend = arch, layer_idx, attn_backend
        H, D, std = arch.hidden_size, arch.head_dim, arch.initializer_range
        self.nq, self.nkv, self.D = arch.num_attention_heads, arch.num_key_value_heads, D
        self.q_proj = Linear(H, self.nq * D * 2, bias=arch.attention_bias, std=std, dtype=dtype, device=device)
        self.k_proj = Linear(H, self.nkv * D, bias=arch.attention_bias, std=std, dtype=dtype, device=device)
        self.v_proj = Linear(H, self.nkv * D, bias=arch.attention_bias, std=std, dtype=dtype, device=device)
        self.o_proj = Linear(self.nq * D, H, bias=arch.attention_bias, std=std, dtype=dtype, device=device)
        self.q_norm = RMSNorm(D, arch.rms_norm_eps, dtype=dtype, device=device)
        self.k_norm = RMSNorm(D, arch.rms_norm_eps, dtype=dtype, device=device)
        self.register_buffer("inv_freq", ops.inv_freq(D, arch.rope_theta, device=device, rotary_dim=arch.rotary_dim),
                             persistent=False)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        T = x.shape[0]
        qg = self.q_proj(x).view(T, self.nq, 2 * self.D)
        q, gate = qg[..., : self.D], qg[..., self.D:]
        k = self.k_proj(x).view(T, self.nkv, self.D)
        v = self.v_proj(x).view(T, self.nkv, self.D)
        if seq.mrope_angles is not None:
            q = norm_rope_with_angles(q, self.q_norm.weight, seq.mrope_angles, self.arch.rms_norm_eps)
            k = norm_rope_with_angles(k, self.k_norm.weight, seq.mrope_angles, self.arch.rms_norm_eps)
        else:
            q = ops.qknorm_rope(q, self.q_norm.weight, seq.position_ids, self.inv_freq, self.arch.rms_norm_eps)
            k = ops.qknorm_rope(k, self.k_norm.weight, seq.position_ids, self.inv_freq, self.arch.rms_norm_eps)
        if seq.engine is not None:
            o = seq.engine.attend(self.layer_idx, q, k, v, None, None)
        elif seq.cp is not None:
            o = seq.cp.attention(q, k, v, seq, backend=self.backend)
        else:
            o = attn_ops.attention(q, k, v, seq.cu_seqlens, seq.max_seqlen, causal=True, backend=self.backend,
                                   cache=seq.attn_cache, cache_key=self.layer_idx)
        o = o * torch.sigmoid(gate.float()).to(o.dtype)
        return self.o_proj(o.reshape(T, self.nq * self.D))


def _deinterleave(x: torch.Tensor) -> torch.Tensor:
    """(x0, x1, x2, x3, ...) -> (x0, x2, ..., x1, x3, ...): pairs stored interleaved become the
    two halves that the rotary kernel rotates."""
    d = x.shape[-1]
    return x.reshape(*x.shape[:-1], d // 2, 2).transpose(-1, -2).reshape(*x.shape[:-1], d)


class DSAIndexer(nn.Module):
    def __init__(self, arch: ModelArch, dtype=None, device=None):
        super().__init__()
        self.nh, self.hd, self.rope = arch.index_n_heads, arch.index_head_dim, arch.qk_rope_head_dim
        std = arch.initializer_range
        self.wq_b = Linear(arch.q_lora_rank, self.nh * self.hd, std=std, dtype=dtype, device=device)
        self.wk = Linear(arch.hidden_size, self.hd, bias=arch.attention_bias, std=std, dtype=dtype, device=device)
        self.k_norm = nn.LayerNorm(self.hd, eps=1e-6, dtype=dtype, device=device)
        self.weights_proj = Linear(arch.hidden_size, self.nh, std=std, dtype=dtype, device=device)
        for p in self.parameters():         # the selection carries no gradient (as in the reference)
            p.requires_grad_(False)

    @torch.no_grad()
    def project(self, x, q_latent, seq: SeqInfo, inv_freq):
        """Indexer queries ``[T, Hi, Di]``, keys ``[T, Di]`` (both rotated) and head weights ``[T, Hi]`` of the tokens."""
        T = x.shape[0]
        q = self.wq_b(q_latent).view(T, self.nh, self.hd)
        k = self.k_norm(self.wk(x)).view(T, 1, self.hd)
        w = self.weights_proj(x)

        def rope_head(t):
            pe = ops.qknorm_rope(_deinterleave(t[..., : self.rope]).contiguous(), None, seq.position_ids, inv_freq)
            return torch.cat([pe, t[..., self.rope:]], dim=-1)

        return rope_head(q), rope_head(k)[:, 0], w

    @torch.no_grad()
    def forward(self, x, q_latent, seq: SeqInfo, inv_freq, topk: int) -> torch.Tensor:
        q, k, w = self.project(x, q_latent, seq, inv_freq)
        ks, ke = doc_windows(seq)
        return sparse_mla.dsa_indexer_topk(q, k, w, ks, ke, topk)


class SparseMLAAttention(nn.Module):
    """Multi-head latent attention in absorbed form over the top-k keys the indexer selects.
    ``share_indices``: the layer reuses the selection of the closest earlier layer that has an
    indexer (kept on ``seq`` for the duration of one forward)."""

    def __init__(self, arch: ModelArch, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.arch, self.layer_idx = arch, layer_idx
        a, std = arch, arch.initializer_range
        self.nh = a.num_attention_heads
        self.qk_head_dim = a.qk_nope_head_dim + a.qk_rope_head_dim
        self.q_a_proj = Linear(a.hidden_size, a.q_lora_rank, bias=a.attention_bias, std=std, dtype=dtype, device=device)
        self.q_a_layernorm = RMSNorm(a.q_lora_rank, a.rms_norm_eps, dtype=dtype, device=device)
        self.q_b_proj = Linear(a.q_lora_rank, self.nh * self.qk_head_dim, std=std, dtype=dtype, device=device)
        self.kv_a_proj_with_mqa = Linear(a.hidden_size, a.kv_lora_rank + a.qk_rope_head_dim, bias=a.attention_bias,
                                         std=std, dtype=dtype, device=device)
        self.kv_a_layernorm = RMSNorm(a.kv_lora_rank, a.rms_norm_eps, dtype=dtype, device=device)
        self.kv_b_proj = Linear(a.kv_lora_rank, self.nh * (a.qk_nope_head_dim + a.v_head_dim), std=std, dtype=dtype,
                                device=device)
        self.o_proj = Linear(self.nh * a.v_head_dim, a.hidden_size, bias=a.attention_bias, std=std, dtype=dtype,
                             device=device)
        self.skip_topk = bool(a.index_share_layers and layer_idx in a.index_share_layers)
        self.indexer = None if self.skip_topk else DSAIndexer(a, dtype=dtype, device=device)
        # the layer whose selection this one uses (itself, or the closest earlier layer with an indexer)
        self.index_source = layer_idx
        while self.index_source in (a.index_share_layers or []):
            self.index_source -= 1
        self.scaling = self.qk_head_dim ** -0.5
        self.register_buffer("inv_freq", ops.inv_freq(a.qk_rope_head_dim, a.rope_theta, device=device), persistent=False)

    def forward(self, x: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        a, T = self.arch, x.shape[0]
        q_latent = self.q_a_layernorm(self.q_a_proj(x))
        ckv, k_rope = self.kv_a_proj_with_mqa(x).split([a.kv_lora_rank, a.qk_rope_head_dim], dim=-1)
        ckv = self.kv_a_layernorm(ckv.contiguous())
        if seq.engine is not None:
            return self._forward_engine(x, seq, q_latent, ckv, k_rope)
        if seq.cp is not None:
            return self._forward_cp(x, seq, q_latent, ckv, k_rope)
        if self.indexer is not None:
            indices = self.indexer(x, q_latent, seq, self.inv_freq, a.index_topk)
            if seq.shared is None:
                seq.shared = {}
            seq.shared[("dsa", self.layer_idx)] = indices
        else:
            indices = (seq.shared or {}).get(("dsa", self.index_source))
            if indices is None:
                raise RuntimeError("a layer that shares sparse indices ran before the layer that computes them")
        sq, skv, w_v = self._absorbed(q_latent, ckv, k_rope, seq)
        o = sparse_mla.sparse_mla_attention(sq, skv, indices, self.scaling, a.kv_lora_rank)
        o = torch.einsum("thk,hdk->thd", o, w_v)                    # value up-projection per head
        return self.o_proj(o.reshape(T, self.nh * a.v_head_dim))

    def _absorbed(self, q_latent, ckv, k_rope, seq: SeqInfo):
        """Queries with the key up-projection absorbed ``[T, H, rank + rope]``, the tokens' latent K / V rows
        ``[T, rank + rope]`` and the value up-projection ``[H, dv, rank]``."""
        a, T = self.arch, q_latent.shape[0]
        q = self.q_b_proj(q_latent).view(T, self.nh, self.qk_head_dim)
        q_nope, q_rope = q[..., : a.qk_nope_head_dim], q[..., a.qk_nope_head_dim:]
        q_rope = ops.qknorm_rope(_deinterleave(q_rope).contiguous(), None, seq.position_ids, self.inv_freq)
        k_rope = ops.qknorm_rope(_deinterleave(k_rope).reshape(T, 1, -1).contiguous(), None, seq.position_ids,
                                 self.inv_freq)[:, 0]
        w = self.kv_b_proj.weight.view(self.nh, a.qk_nope_head_dim + a.v_head_dim, a.kv_lora_rank)
        w_k, w_v = w[:, : a.qk_nope_head_dim], w[:, a.qk_nope_head_dim:]
        q_abs = torch.einsum("thd,hdk->thk", q_nope, w_k)          # absorb the key up-projection into q
        return torch.cat([q_abs, q_rope], dim=-1), torch.cat([ckv, k_rope], dim=-1), w_v

    def _forward_cp(self, x, seq: SeqInfo, q_latent, ckv, k_rope) -> torch.Tensor:
        """Context parallelism: the latent K / V rows (and the indexer keys) are small per token, so they are gathered
        whole; the local queries select and attend over the global sequence (reference: all-gather of the compressed
        K / V, src/prime_rl/trainer/models/glm_moe_dsa/sparse_mla_attention.py:208-210)."""
        a, T, cp = self.arch, x.shape[0], seq.cp
        sq, skv, w_v = self._absorbed(q_latent, ckv, k_rope, seq)
        skv_all = cp.gather_rows(skv)
        rows = cp.global_rows(T, x.device)
        if self.indexer is not None:
            q_i, k_i, w_i = self.indexer.project(x, q_latent, seq, self.inv_freq)
            k_all = cp.gather_rows(k_i, grad=False)
            ke = (rows + 1).to(torch.int32)
            ks = (rows - seq.position_ids.to(rows.dtype)).to(torch.int32)          # first token of the row's document
            indices = sparse_mla.dsa_indexer_topk(q_i, k_all, w_i, ks, ke, a.index_topk)
            if seq.shared is None:
                seq.shared = {}
            seq.shared[("dsa", self.layer_idx)] = indices
        else:
            indices = (seq.shared or {}).get(("dsa", self.index_source))
            if indices is None:
                raise RuntimeError("a layer that shares sparse indices ran before the layer that computes them")
        o = sparse_mla.sparse_mla_attention(sq, skv_all, indices, self.scaling, a.kv_lora_rank)
        o = torch.einsum("thk,hdk->thd", o, w_v)
        return self.o_proj(o.reshape(T, self.nh * a.v_head_dim))

    def _forward_engine(self, x, seq: SeqInfo, q_latent, ckv, k_rope) -> torch.Tensor:
        """Rollout engine: the latent K / V rows and the indexer keys of earlier tokens come from the engine's
        per-sequence store (``engine/hybrid.py: RecurrentStep.sparse_mla``)."""
        a, T = self.arch, x.shape[0]
        sq, skv, w_v = self._absorbed(q_latent, ckv, k_rope, seq)
        idx_in = self.indexer.project(x, q_latent, seq, self.inv_freq) if self.indexer is not None else None
        o = seq.engine.sparse_mla(self.layer_idx, self.index_source, sq, skv, idx_in, a.index_topk, self.scaling,
                                  a.kv_lora_rank)
        o = torch.einsum("thk,hdk->thd", o, w_v)
        return self.o_proj(o.reshape(T, self.nh * a.v_head_dim))
