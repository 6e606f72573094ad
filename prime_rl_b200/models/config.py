"""Architecture description shared by the trainer models and the rollout engine.

One ``ModelArch`` covers the supported decoder families; ``from_hf_config`` reads a
HuggingFace ``config.json`` dict (llama, qwen2, qwen3, qwen3_moe, glm4_moe, gpt_oss,
minimax_m2, afmoe) and ``to_hf_config`` writes one back for exported checkpoints.
The reference keeps one configuration class per family
(src/prime_rl/trainer/models/*/configuration_*.py); here a family is a set of flags.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict


class ModelArch(BaseModel):
    model_config = ConfigDict(extra="ignore")

    model_type: str = "qwen3"
    vocab_size: int = 151936
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = True                       # per-head RMSNorm on q and k (Qwen3 family)
    hidden_act: Literal["silu", "swiglu_clamped", "relu2", "silu_clamped"] = "silu"
    swiglu_limit: float = 7.0
    swiglu_alpha: float = 1.702
    # attention pattern
    sliding_window: int | None = None
    layer_types: list[str] | None = None       # per layer "full_attention" | "sliding_attention"
    attention_sinks: bool = False              # learnable per-head sink logit (GPT-OSS)
    attn_gate: Literal["none", "per_head", "per_element"] = "none"   # softplus output gate (Laguna)
    heads_per_layer: list[int] | None = None   # query heads of every layer when they differ (Laguna)
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    score_func: Literal["softmax", "sigmoid"] = "softmax"
    routed_scaling_factor: float = 1.0
    router_bias: bool = False                  # selection bias (e_score_correction_bias)
    router_linear_bias: bool = False           # bias term of the gate projection (GPT-OSS)
    expert_bias: bool = False                  # per-expert projection biases (GPT-OSS)
    n_shared_experts: int = 0
    first_k_dense_replace: int = 0             # first k layers use a dense MLP
    mlp_only_layers: list[int] = []
    mlp_layer_types: list[str] | None = None   # per layer "dense" | "sparse" (overrides the rules below)
    shared_expert_intermediate_size: int = 0   # width of the shared expert when it differs from moe_intermediate_size
    decoder_sparse_step: int = 1
    initializer_range: float = 0.02
    final_logit_softcapping: float | None = None   # softcap * tanh(z / softcap) on the output logits (Gemma)
    shared_expert_gate: bool = False           # sigmoid gate on the shared expert's output (Qwen3.5-MoE)
    moe_latent_size: int = 0                   # experts work in a projected space of this width (Nemotron-H)
    # layer kinds. block_types: every layer is ONE pre-normed mixer ("mamba" | "attention" | "mlp" | "moe",
    # Nemotron-H); mixer_types: token mixer of a standard two-sublayer block ("attention" | "gated_attention" |
    # "gated_delta_net" | "mla_dsa")
    block_types: list[str] | None = None
    mixer_types: list[str] | None = None
    use_rope: bool = True
    # Mamba-2
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    ssm_state_size: int = 0
    ssm_n_groups: int = 1
    conv_kernel: int = 4
    ssm_chunk_size: int = 128
    mamba_proj_bias: bool = False
    use_conv_bias: bool = True
    time_step_limit: tuple[float, float] = (0.0, float("inf"))
    # gated delta-net
    linear_num_value_heads: int = 0
    linear_num_key_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    # multi-head latent attention + sparse indexer
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_rope_head_dim: int = 0
    qk_nope_head_dim: int = 0
    v_head_dim: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    index_share_layers: list[int] = []        # layers without an indexer: they reuse the previous selection
    # DeepSeek-V4: hyper-connection streams, compressed attention, grouped output projection, hash-routed layers
    hc_mult: int = 0
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    csa_compress_rate: int = 0                # "compressed_sparse_attention" layers
    hca_compress_rate: int = 0                # "heavily_compressed_attention" layers
    compress_rope_theta: float = 160000.0
    o_groups: int = 1
    o_lora_rank: int = 0
    num_hash_layers: int = 0

    # ------------------------------------------------------------------ derived
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def block_type(self, idx: int) -> str:
        return self.block_types[idx] if self.block_types is not None else "standard"

    def mixer_type(self, idx: int) -> str:
        return self.mixer_types[idx] if self.mixer_types is not None else "attention"

    @property
    def expert_hidden(self) -> int:
        return self.moe_latent_size or self.hidden_size

    def layer_is_moe(self, idx: int) -> bool:
        if self.block_types is not None:
            return self.block_types[idx] == "moe"
        if self.is_moe and self.mlp_layer_types is not None:
            return self.mlp_layer_types[idx] == "sparse"
        if not self.is_moe or idx in self.mlp_only_layers or idx < self.first_k_dense_replace:
            return False
        return (idx + 1) % self.decoder_sparse_step == 0

    def layer_window(self, idx: int) -> int | None:
        if self.sliding_window is None:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[idx] == "sliding_attention" else None

    def layer_heads(self, idx: int) -> int:
        return self.heads_per_layer[idx] if self.heads_per_layer is not None else self.num_attention_heads

    @property
    def shared_width(self) -> int:
        return self.shared_expert_intermediate_size or self.moe_intermediate_size * self.n_shared_experts

    @property
    def rotary_dim(self) -> int:
        rd = int(self.head_dim * self.partial_rotary_factor)
        return rd - rd % 2

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def param_count(self, active_only: bool = False, matmul_only: bool = False) -> int:
        """Parameter count; ``active_only`` counts top-k experts instead of all of them and
        ``matmul_only`` leaves out embeddings and norms (the MFU formula's convention)."""
        H = self.hidden_size
        attn = H * (self.q_dim + 2 * self.kv_dim) + self.q_dim * H
        dense_mlp = 3 * H * self.intermediate_size
        expert = 3 * H * self.moe_intermediate_size
        total = 0
        for i in range(self.num_hidden_layers):
            bt, mt = self.block_type(i), self.mixer_type(i)
            if bt == "mamba":
                inner = self.mamba_num_heads * self.mamba_head_dim
                conv = inner + 2 * self.ssm_n_groups * self.ssm_state_size
                total += H * (inner + conv + self.mamba_num_heads) + inner * H
                continue
            if bt in ("mlp", "moe"):
                pass
            elif mt == "gated_delta_net":
                kd, vd = self.linear_num_key_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
                total += H * (2 * kd + 2 * vd + 2 * self.linear_num_value_heads) + vd * H
            elif mt == "mla_dsa":
                qk = self.qk_nope_head_dim + self.qk_rope_head_dim
                total += (H * self.q_lora_rank + self.q_lora_rank * self.num_attention_heads * qk
                          + H * (self.kv_lora_rank + self.qk_rope_head_dim)
                          + self.kv_lora_rank * self.num_attention_heads * (self.qk_nope_head_dim + self.v_head_dim)
                          + self.num_attention_heads * self.v_head_dim * H)
            elif mt == "gated_attention":
                total += attn + H * self.q_dim
            else:
                total += attn
            if bt == "attention":
                continue
            if bt == "mlp":
                total += (2 if self.hidden_act == "relu2" else 3) * H * self.intermediate_size
                continue
            if self.layer_is_moe(i):
                n = self.num_experts_per_tok if active_only else self.num_experts
                total += n * expert + H * self.num_experts + self.n_shared_experts * expert
            else:
                total += dense_mlp
            if not matmul_only:
                total += 2 * H + (2 * self.head_dim if self.qk_norm else 0)
        total += self.vocab_size * H  # lm head
        if not matmul_only:
            total += H + (0 if self.tie_word_embeddings else self.vocab_size * H)
        return total

    # ------------------------------------------------------------------ HF interchange
    @classmethod
    def from_hf_config(cls, cfg: dict[str, Any]) -> "ModelArch":
        mt = cfg.get("model_type", "llama")
        if mt in ("qwen3_5", "qwen3_5_moe") and "text_config" in cfg:      # multimodal wrapper: the text tower
            cfg = {**cfg["text_config"], "model_type": mt}
        mt = {"qwen3_5_text": "qwen3_5", "qwen3_5_moe_text": "qwen3_5_moe"}.get(mt, mt)
        # transformers >= 5 writes some fields under other names (``num_local_experts`` for ``num_experts``,
        # ``rope_parameters`` for ``rope_theta`` / ``rope_scaling``): accept both spellings
        cfg = dict(cfg)
        for ours, theirs in (("num_experts", "num_local_experts"), ("num_local_experts", "num_experts")):
            if ours not in cfg and theirs in cfg:
                cfg[ours] = cfg[theirs]
        heads = cfg["num_attention_heads"]
        d: dict[str, Any] = dict(
            model_type=mt,
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            num_hidden_layers=cfg["num_hidden_layers"],
            num_attention_heads=heads,
            num_key_value_heads=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            intermediate_size=cfg.get("intermediate_size", 0),
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
            rope_theta=cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta", 1e4),
            partial_rotary_factor=cfg.get("partial_rotary_factor") or
            (cfg.get("rope_parameters") or {}).get("partial_rotary_factor", 1.0),
            max_position_embeddings=cfg.get("max_position_embeddings", 32768),
            tie_word_embeddings=cfg.get("tie_word_embeddings", False),
            attention_bias=cfg.get("attention_bias", False),
            sliding_window=cfg.get("sliding_window") if cfg.get("use_sliding_window", True) else None,
            layer_types=cfg.get("layer_types"),
            initializer_range=cfg.get("initializer_range", 0.02),
        )
        if mt in ("llama", "mistral"):
            d.update(qk_norm=False)
        elif mt == "qwen2":
            d.update(qk_norm=False, attention_bias=True, sliding_window=None)
        elif mt == "qwen3":
            d.update(qk_norm=True, sliding_window=None)
        elif mt == "qwen3_moe":
            d.update(qk_norm=True, sliding_window=None, num_experts=cfg["num_experts"],
                     num_experts_per_tok=cfg["num_experts_per_tok"],
                     moe_intermediate_size=cfg["moe_intermediate_size"],
                     norm_topk_prob=cfg.get("norm_topk_prob", True),
                     mlp_only_layers=cfg.get("mlp_only_layers", []),
                     decoder_sparse_step=cfg.get("decoder_sparse_step", 1))
        elif mt == "glm4_moe":
            d.update(qk_norm=cfg.get("use_qk_norm", False), num_experts=cfg["n_routed_experts"],
                     num_experts_per_tok=cfg["num_experts_per_tok"],
                     moe_intermediate_size=cfg["moe_intermediate_size"],
                     norm_topk_prob=cfg.get("norm_topk_prob", True), score_func="sigmoid", router_bias=True,
                     routed_scaling_factor=cfg.get("routed_scaling_factor", 1.0),
                     n_shared_experts=cfg.get("n_shared_experts", 1),
                     first_k_dense_replace=cfg.get("first_k_dense_replace", 0), sliding_window=None)
        elif mt == "gpt_oss":
            d.update(qk_norm=False, attention_bias=True, attention_sinks=True, hidden_act="swiglu_clamped",
                     swiglu_limit=cfg.get("swiglu_limit", 7.0), num_experts=cfg["num_local_experts"],
                     num_experts_per_tok=cfg.get("num_experts_per_tok", cfg.get("experts_per_token", 4)),
                     moe_intermediate_size=cfg["intermediate_size"], norm_topk_prob=True,
                     router_linear_bias=True, expert_bias=True)
        elif mt == "minimax_m2":
            d.update(qk_norm=True, num_experts=cfg["num_local_experts"],
                     num_experts_per_tok=cfg["num_experts_per_tok"], moe_intermediate_size=cfg["intermediate_size"],
                     score_func="sigmoid", router_bias=True, sliding_window=None)
        elif mt == "afmoe":
            d.update(qk_norm=True, num_experts=cfg["num_experts"], num_experts_per_tok=cfg["num_experts_per_tok"],
                     moe_intermediate_size=cfg["moe_intermediate_size"], score_func="sigmoid", router_bias=True,
                     n_shared_experts=cfg.get("num_shared_experts", 0),
                     first_k_dense_replace=cfg.get("num_dense_layers", 0),
                     routed_scaling_factor=cfg.get("route_scale", 1.0))
        elif mt == "laguna":
            gating = cfg.get("gating", True)
            n = cfg["num_hidden_layers"]
            d.update(qk_norm=True, num_experts=cfg.get("num_experts", cfg.get("num_local_experts", 0)),
                     num_experts_per_tok=cfg["num_experts_per_tok"],
                     moe_intermediate_size=cfg["moe_intermediate_size"], score_func="sigmoid", norm_topk_prob=True,
                     router_bias=True, routed_scaling_factor=cfg.get("moe_routed_scaling_factor", 1.0),
                     n_shared_experts=1, shared_expert_intermediate_size=cfg.get("shared_expert_intermediate_size", 0),
                     mlp_layer_types=cfg.get("mlp_layer_types") or ["sparse"] * n,
                     heads_per_layer=cfg.get("num_attention_heads_per_layer"),
                     attn_gate="none" if not gating else ("per_head" if gating == "per-head" else "per_element"))
        elif mt == "nemotron_h":
            kinds = {"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}
            blocks = cfg.get("layers_block_type") or [kinds[c] for c in cfg.get("hybrid_override_pattern", "ME*E")]
            d.update(num_hidden_layers=len(blocks), block_types=blocks, qk_norm=False, use_rope=False,
                     hidden_act=cfg.get("mlp_hidden_act", "relu2"), rms_norm_eps=cfg.get("layer_norm_epsilon", 1e-5),
                     mamba_num_heads=cfg.get("mamba_num_heads", 128), mamba_head_dim=cfg.get("mamba_head_dim", 64),
                     ssm_state_size=cfg.get("ssm_state_size", 128), ssm_n_groups=cfg.get("n_groups", 8),
                     conv_kernel=cfg.get("conv_kernel", 4), ssm_chunk_size=cfg.get("chunk_size", 128),
                     mamba_proj_bias=cfg.get("use_bias", False), use_conv_bias=cfg.get("use_conv_bias", True),
                     time_step_limit=tuple(cfg.get("time_step_limit") or (0.0, float("inf"))), sliding_window=None)
            if "moe" in blocks:
                d.update(num_experts=cfg.get("n_routed_experts", 8), num_experts_per_tok=cfg.get("num_experts_per_tok", 2),
                         moe_intermediate_size=cfg.get("moe_intermediate_size", 0), score_func="sigmoid",
                         router_bias=True, norm_topk_prob=cfg.get("norm_topk_prob", True),
                         routed_scaling_factor=cfg.get("routed_scaling_factor", 1.0), n_shared_experts=1,
                         shared_expert_intermediate_size=cfg.get("moe_shared_expert_intermediate_size", 0),
                         moe_latent_size=cfg.get("moe_latent_size") or 0)
        elif mt in ("qwen3_5", "qwen3_5_moe"):
            n = cfg["num_hidden_layers"]
            every = cfg.get("full_attention_interval", 4)
            kinds = cfg.get("layer_types") or ["full_attention" if (i + 1) % every == 0 else "linear_attention"
                                               for i in range(n)]
            rope = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
            d.update(qk_norm=True, sliding_window=None, layer_types=None,
                     mixer_types=["gated_attention" if k == "full_attention" else "gated_delta_net" for k in kinds],
                     partial_rotary_factor=rope.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 0.25)),
                     rope_theta=rope.get("rope_theta", cfg.get("rope_theta", 1e4)),
                     linear_num_value_heads=cfg.get("linear_num_value_heads", 32),
                     linear_num_key_heads=cfg.get("linear_num_key_heads", 16),
                     linear_key_head_dim=cfg.get("linear_key_head_dim", 128),
                     linear_value_head_dim=cfg.get("linear_value_head_dim", 128),
                     linear_conv_kernel_dim=cfg.get("linear_conv_kernel_dim", 4))
            if mt == "qwen3_5_moe":
                d.update(num_experts=cfg["num_experts"], num_experts_per_tok=cfg["num_experts_per_tok"],
                         moe_intermediate_size=cfg["moe_intermediate_size"], norm_topk_prob=True, n_shared_experts=1,
                         shared_expert_intermediate_size=cfg.get("shared_expert_intermediate_size", 0),
                         shared_expert_gate=True)
        elif mt == "deepseek_v4":
            n = cfg["num_hidden_layers"]
            rates = cfg.get("compress_rates") or {}
            kinds = cfg.get("layer_types")
            if kinds is None:
                inter = ["compressed_sparse_attention" if i % 2 == 0 else "heavily_compressed_attention"
                         for i in range(max(n - 2, 0))]
                kinds = (["heavily_compressed_attention"] * min(n, 2) + inter)[:n]
            hd = cfg.get("head_dim", 512)
            d.update(qk_norm=False, head_dim=hd, num_key_value_heads=1, layer_types=kinds,
                     sliding_window=cfg.get("sliding_window", 128), hidden_act="silu_clamped",
                     swiglu_limit=cfg.get("swiglu_limit", 10.0), q_lora_rank=cfg["q_lora_rank"],
                     qk_rope_head_dim=cfg.get("qk_rope_head_dim") or int(hd * cfg.get("partial_rotary_factor", 0.125)),
                     compress_rope_theta=cfg.get("compress_rope_theta", 160000.0),
                     csa_compress_rate=rates.get("compressed_sparse_attention", 4),
                     hca_compress_rate=rates.get("heavily_compressed_attention", 128),
                     index_n_heads=cfg.get("index_n_heads", 64), index_head_dim=cfg.get("index_head_dim", 128),
                     index_topk=cfg.get("index_topk", 512), o_groups=cfg.get("o_groups", 8),
                     o_lora_rank=cfg.get("o_lora_rank", 1024), num_hash_layers=cfg.get("num_hash_layers", 3),
                     hc_mult=cfg.get("hc_mult", 4), hc_sinkhorn_iters=cfg.get("hc_sinkhorn_iters", 20),
                     hc_eps=cfg.get("hc_eps", 1e-6), num_experts=cfg["n_routed_experts"],
                     num_experts_per_tok=cfg["num_experts_per_tok"], moe_intermediate_size=cfg["moe_intermediate_size"],
                     norm_topk_prob=True, score_func="sigmoid", router_bias=True,
                     routed_scaling_factor=cfg.get("routed_scaling_factor", 1.0),
                     n_shared_experts=1 if cfg.get("n_shared_experts", 1) > 0 else 0)
        elif mt == "glm_moe_dsa":
            n = cfg["num_hidden_layers"]
            d.update(qk_norm=False, sliding_window=None, mixer_types=["mla_dsa"] * n,
                     kv_lora_rank=cfg["kv_lora_rank"], q_lora_rank=cfg["q_lora_rank"],
                     qk_rope_head_dim=cfg["qk_rope_head_dim"], qk_nope_head_dim=cfg["qk_nope_head_dim"],
                     v_head_dim=cfg["v_head_dim"], index_n_heads=cfg.get("index_n_heads", 32),
                     index_head_dim=cfg.get("index_head_dim", 128), index_topk=cfg.get("index_topk", 2048),
                     index_share_layers=cfg.get("index_share_layers") or [],
                     num_experts=cfg["n_routed_experts"], num_experts_per_tok=cfg["num_experts_per_tok"],
                     moe_intermediate_size=cfg["moe_intermediate_size"], norm_topk_prob=cfg.get("norm_topk_prob", True),
                     score_func="sigmoid", router_bias=True, routed_scaling_factor=cfg.get("routed_scaling_factor", 1.0),
                     n_shared_experts=cfg.get("n_shared_experts", 1),
                     first_k_dense_replace=cfg.get("first_k_dense_replace", 0))
        else:
            raise ValueError(f"unsupported model_type '{mt}'")
        return cls(**d)

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "ModelArch":
        return cls.from_hf_config(json.loads((Path(path) / "config.json").read_text()))

    def to_hf_config(self) -> dict[str, Any]:
        arch_names = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                      "qwen3_moe": "Qwen3MoeForCausalLM", "glm4_moe": "Glm4MoeForCausalLM",
                      "gpt_oss": "GptOssForCausalLM", "minimax_m2": "MiniMaxM2ForCausalLM",
                      "afmoe": "AfmoeForCausalLM", "laguna": "LagunaForCausalLM",
                      "nemotron_h": "NemotronHForCausalLM", "qwen3_5": "Qwen3_5ForCausalLM",
                      "qwen3_5_moe": "Qwen3_5MoeForCausalLM", "glm_moe_dsa": "GlmMoeDsaForCausalLM",
                      "deepseek_v4": "DeepseekV4ForCausalLM"}
        cfg: dict[str, Any] = dict(
            architectures=[arch_names.get(self.model_type, "LlamaForCausalLM")], model_type=self.model_type,
            vocab_size=self.vocab_size, hidden_size=self.hidden_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim, intermediate_size=self.intermediate_size, rms_norm_eps=self.rms_norm_eps,
            rope_theta=self.rope_theta, max_position_embeddings=self.max_position_embeddings,
            tie_word_embeddings=self.tie_word_embeddings, attention_bias=self.attention_bias,
            hidden_act="silu", torch_dtype="bfloat16", initializer_range=self.initializer_range)
        if self.is_moe:
            if self.model_type == "glm4_moe":
                cfg.update(n_routed_experts=self.num_experts, n_shared_experts=self.n_shared_experts,
                           first_k_dense_replace=self.first_k_dense_replace,
                           routed_scaling_factor=self.routed_scaling_factor, use_qk_norm=self.qk_norm)
            elif self.model_type in ("gpt_oss", "minimax_m2"):
                cfg.update(num_local_experts=self.num_experts)
            elif self.model_type == "laguna":
                gating = {"none": False, "per_head": "per-head", "per_element": True}[self.attn_gate]
                cfg.update(num_experts=self.num_experts, mlp_layer_types=self.mlp_layer_types, gating=gating,
                           shared_expert_intermediate_size=self.shared_width,
                           num_attention_heads_per_layer=self.heads_per_layer or
                           [self.num_attention_heads] * self.num_hidden_layers,
                           moe_routed_scaling_factor=self.routed_scaling_factor)
            else:
                cfg.update(num_experts=self.num_experts, mlp_only_layers=self.mlp_only_layers,
                           decoder_sparse_step=self.decoder_sparse_step)
            cfg.update(num_experts_per_tok=self.num_experts_per_tok,
                       moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob)
        if self.sliding_window is not None:
            cfg.update(sliding_window=self.sliding_window, layer_types=self.layer_types)
        if self.model_type == "nemotron_h":
            cfg.update(layers_block_type=self.block_types, mlp_hidden_act=self.hidden_act,
                       layer_norm_epsilon=self.rms_norm_eps, mamba_num_heads=self.mamba_num_heads,
                       mamba_head_dim=self.mamba_head_dim, ssm_state_size=self.ssm_state_size,
                       n_groups=self.ssm_n_groups, conv_kernel=self.conv_kernel, chunk_size=self.ssm_chunk_size,
                       use_bias=self.mamba_proj_bias, use_conv_bias=self.use_conv_bias,
                       n_routed_experts=self.num_experts, moe_latent_size=self.moe_latent_size or None,
                       moe_shared_expert_intermediate_size=self.shared_width)
        elif self.model_type in ("qwen3_5", "qwen3_5_moe"):
            cfg.update(layer_types=["full_attention" if m == "gated_attention" else "linear_attention"
                                    for m in (self.mixer_types or [])],
                       partial_rotary_factor=self.partial_rotary_factor,
                       linear_num_value_heads=self.linear_num_value_heads,
                       linear_num_key_heads=self.linear_num_key_heads, linear_key_head_dim=self.linear_key_head_dim,
                       linear_value_head_dim=self.linear_value_head_dim,
                       linear_conv_kernel_dim=self.linear_conv_kernel_dim,
                       shared_expert_intermediate_size=self.shared_width)
        elif self.model_type == "deepseek_v4":
            cfg.update(layer_types=self.layer_types, sliding_window=self.sliding_window, swiglu_limit=self.swiglu_limit,
                       q_lora_rank=self.q_lora_rank, qk_rope_head_dim=self.qk_rope_head_dim,
                       compress_rope_theta=self.compress_rope_theta,
                       compress_rates={"compressed_sparse_attention": self.csa_compress_rate,
                                       "heavily_compressed_attention": self.hca_compress_rate},
                       index_n_heads=self.index_n_heads, index_head_dim=self.index_head_dim, index_topk=self.index_topk,
                       o_groups=self.o_groups, o_lora_rank=self.o_lora_rank, num_hash_layers=self.num_hash_layers,
                       hc_mult=self.hc_mult, hc_sinkhorn_iters=self.hc_sinkhorn_iters, hc_eps=self.hc_eps,
                       n_routed_experts=self.num_experts, n_shared_experts=self.n_shared_experts,
                       routed_scaling_factor=self.routed_scaling_factor)
        elif self.model_type == "glm_moe_dsa":
            cfg.update(kv_lora_rank=self.kv_lora_rank, q_lora_rank=self.q_lora_rank,
                       qk_rope_head_dim=self.qk_rope_head_dim, qk_nope_head_dim=self.qk_nope_head_dim,
                       v_head_dim=self.v_head_dim, index_n_heads=self.index_n_heads,
                       index_head_dim=self.index_head_dim, index_topk=self.index_topk,
                       index_share_layers=self.index_share_layers, n_routed_experts=self.num_experts,
                       n_shared_experts=self.n_shared_experts, first_k_dense_replace=self.first_k_dense_replace,
                       routed_scaling_factor=self.routed_scaling_factor)
        return cfg


# Shapes named by the benchmarks and examples (random-init; no download needed).
PRESETS: dict[str, dict[str, Any]] = {
    "qwen3-0.6b": dict(model_type="qwen3", hidden_size=1024, num_hidden_layers=28, num_attention_heads=16,
                       num_key_value_heads=8, head_dim=128, intermediate_size=3072, tie_word_embeddings=True),
    "qwen3-4b": dict(model_type="qwen3", hidden_size=2560, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=9728, tie_word_embeddings=True),
    "qwen3-8b": dict(model_type="qwen3", hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=12288),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", hidden_size=2048, num_hidden_layers=48, num_attention_heads=32,
                          num_key_value_heads=4, head_dim=128, intermediate_size=6144, num_experts=128,
                          num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True),
    "tiny-laguna": dict(model_type="laguna", hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=512, qk_norm=True,
                        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, score_func="sigmoid",
                        router_bias=True, n_shared_experts=1, shared_expert_intermediate_size=96,
                        mlp_layer_types=["dense", "sparse", "sparse"], heads_per_layer=[4, 2, 4],
                        sliding_window=16, layer_types=["sliding_attention", "full_attention", "sliding_attention"],
                        attn_gate="per_head", max_position_embeddings=512),
    "tiny-nemotron-h": dict(model_type="nemotron_h", hidden_size=128, num_hidden_layers=4, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=512, qk_norm=False,
                            use_rope=False, hidden_act="relu2", block_types=["mamba", "moe", "attention", "mlp"],
                            mamba_num_heads=8, mamba_head_dim=16, ssm_state_size=16, ssm_n_groups=2, ssm_chunk_size=16,
                            num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, score_func="sigmoid",
                            router_bias=True, n_shared_experts=1, shared_expert_intermediate_size=96,
                            moe_latent_size=64, rms_norm_eps=1e-5, max_position_embeddings=512),
    "tiny-qwen3.5-moe": dict(model_type="qwen3_5_moe", hidden_size=128, num_hidden_layers=4, num_attention_heads=4,
                             num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=512, qk_norm=True,
                             partial_rotary_factor=0.25, rope_theta=1e4,
                             mixer_types=["gated_delta_net", "gated_delta_net", "gated_delta_net", "gated_attention"],
                             linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                             linear_value_head_dim=16, num_experts=4, num_experts_per_tok=2,
                             moe_intermediate_size=64, n_shared_experts=1, shared_expert_intermediate_size=64,
                             shared_expert_gate=True, max_position_embeddings=512),
    "tiny-glm-moe-dsa": dict(model_type="glm_moe_dsa", hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
                             num_key_value_heads=4, head_dim=32, intermediate_size=256, vocab_size=512, qk_norm=False,
                             mixer_types=["mla_dsa"] * 3, kv_lora_rank=32, q_lora_rank=48, qk_rope_head_dim=16,
                             qk_nope_head_dim=16, v_head_dim=24, index_n_heads=2, index_head_dim=32, index_topk=8,
                             index_share_layers=[2], num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                             score_func="sigmoid", router_bias=True, n_shared_experts=1, first_k_dense_replace=1,
                             max_position_embeddings=512),
    "tiny-deepseek-v4": dict(model_type="deepseek_v4", hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                             num_key_value_heads=1, head_dim=32, intermediate_size=128, vocab_size=256, qk_norm=False,
                             layer_types=["sliding_attention", "heavily_compressed_attention",
                                          "compressed_sparse_attention", "heavily_compressed_attention"],
                             sliding_window=6, hidden_act="silu_clamped", swiglu_limit=10.0, q_lora_rank=24,
                             qk_rope_head_dim=8, csa_compress_rate=2, hca_compress_rate=4, index_n_heads=2,
                             index_head_dim=16, index_topk=4, o_groups=2, o_lora_rank=16, num_hash_layers=1,
                             hc_mult=2, hc_sinkhorn_iters=4, num_experts=4, num_experts_per_tok=2,
                             moe_intermediate_size=32, score_func="sigmoid", router_bias=True, n_shared_experts=1,
                             max_position_embeddings=512),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=64, intermediate_size=512, num_experts=8,
                           num_experts_per_tok=2, moe_intermediate_size=512, vocab_size=4096),
    "tiny-qwen3": dict(model_type="qwen3", hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=4096),
}


def resolve_arch(name_or_path: str, overrides: dict[str, Any] | None = None) -> ModelArch:
    """A preset name, a local HF directory, or inline overrides only."""
    key = name_or_path.lower().split("/")[-1]
    base: dict[str, Any] = {}
    if Path(name_or_path).is_dir() and (Path(name_or_path) / "config.json").exists():
        base = ModelArch.from_pretrained(name_or_path).model_dump()
    else:
        for preset, vals in PRESETS.items():
            if key.startswith(preset) or preset == key:
                base = dict(vals)
                break
        else:
            if not overrides:
                raise FileNotFoundError(
                    f"'{name_or_path}' is neither a local HF directory nor a known preset {sorted(PRESETS)}; "
                    "pass model.arch to describe the architecture inline")
    base.update(overrides or {})
    return ModelArch(**base)
