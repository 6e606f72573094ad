"""Causal LM over packed token streams, with the fused LM head, per-layer activation
recomputation, LoRA injection and freezing helpers.

The forward contract follows the reference's custom models (packed ``[1, T]`` ids with
document boundaries; src/prime_rl/trainer/model.py:1040-1101): ``forward`` returns the
final hidden states, ``logprobs_entropy`` the per-token label log-probabilities and
entropies without materialising logits.
"""

from __future__ import annotations

import re
from typing import Iterable

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from .config import ModelArch
from .layers import DecoderLayer, GroupedExperts, Linear, LoRAAdapter, MoE, MultiLoRA, RMSNorm, SeqInfo


class DecoderStack(nn.Module):
    def __init__(self, arch: ModelArch, attn_backend: str, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(arch.vocab_size, arch.hidden_size, dtype=dtype, device=device)
        layer_cls = DecoderLayer
        if arch.hc_mult:                      # DeepSeek-V4: layers work on [T, hc_mult, hidden] residual streams
            from .deepseek_v4 import DSV4DecoderLayer, HyperHead

            layer_cls = DSV4DecoderLayer
            self.hc_head = HyperHead(arch, dtype=dtype, device=device)
        self.layers = nn.ModuleList(
            [layer_cls(arch, i, attn_backend, dtype=dtype, device=device) for i in range(arch.num_hidden_layers)])
        self.norm = RMSNorm(arch.hidden_size, arch.rms_norm_eps, dtype=dtype, device=device)


class CausalLM(nn.Module):
    def __init__(self, arch: ModelArch, *, attn_backend: str = "auto", dtype=torch.bfloat16, device=None):
        super().__init__()
        self.arch = arch
        self.model = DecoderStack(arch, attn_backend, dtype, device)
        if arch.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = Linear(arch.hidden_size, arch.vocab_size, std=arch.initializer_range, dtype=dtype,
                                  device=device)
        self.ac_every: int | None = None       # recompute every n-th layer in backward (None = never)
        self.cache_attention = True            # keep attention outputs across recomputation
        # "selective" recomputation: operator classes whose outputs are kept as well (ops/stash.py); None = full
        self.ac_keep: set[str] | None = None
        self.layer_hooks = None                # parallel/fsdp.py installs gather/release hooks here

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        """Seeded normal(0, initializer_range) for matrices, ones for norms."""
        gen_dev = next(self.parameters()).device
        gen = torch.Generator(device=gen_dev).manual_seed(seed)
        std = self.arch.initializer_range
        ssm_names = ("A_log", "dt_bias", ".D", "conv1d_weight", "conv1d_bias")
        for name, p in self.named_parameters():
            if "lora_" in name or name.endswith(ssm_names):
                continue
            if name.endswith(("norm.weight", "layernorm.weight", "norm_weight", "hc.scale", "hc_head.hc_scale")):
                p.fill_(1.0)
            elif name.endswith(("hc.base", "hc_head.hc_base", "position_bias")):
                p.zero_()
            elif name.endswith(".bias") or name.endswith("sinks"):
                p.zero_()
            else:
                p.normal_(0.0, std, generator=gen)
        for i, m in enumerate(self.modules()):
            if hasattr(m, "reset_ssm_parameters"):
                m.reset_ssm_parameters(seed=seed * 7919 + i)
        return self

    def full_parameters(self, writeback: bool = False):
        """Context in which every parameter is whole. A no-op for replicated parameters; with parameter
        sharding (``parallel/fsdp.py``) all units are gathered for the duration (a collective: every rank
        enters), and with ``writeback`` values assigned inside are re-sharded on exit (checkpoint load)."""
        import contextlib

        if self.layer_hooks is not None and hasattr(self.layer_hooks, "full_parameters"):
            return self.layer_hooks.full_parameters(writeback=writeback)
        return contextlib.nullcontext()

    @property
    def output_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    # ------------------------------------------------------------------ forward
    def _run_layer(self, layer: DecoderLayer, idx: int, h: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        st = getattr(seq, "op_stash", None)
        if st is not None:                       # selective recomputation: GEMM outputs survive the re-run
            with st.layer(idx):
                return self._run_layer_inner(layer, idx, h, seq)
        return self._run_layer_inner(layer, idx, h, seq)

    def _run_layer_inner(self, layer: DecoderLayer, idx: int, h: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        if self.layer_hooks is not None:
            return self.layer_hooks.run(layer, idx, h, seq)
        return layer(h, seq)

    def forward(self, input_ids: torch.Tensor, seq: SeqInfo, inputs_embeds: torch.Tensor | None = None) -> torch.Tensor:
        """input_ids: [T] (or [1, T]) packed ids -> final hidden states [T, H] (normed).
        ``inputs_embeds [T, H]`` replaces the embedding lookup (multimodal: image features merged in)."""
        ids = input_ids.reshape(-1)
        if self.layer_hooks is not None:
            self.layer_hooks.before_forward()
        h = self.model.embed_tokens(ids) if inputs_embeds is None else inputs_embeds
        if self.arch.hc_mult:
            h = h.unsqueeze(1).expand(-1, self.arch.hc_mult, -1).contiguous()
            seq.shared = dict(seq.shared or {}, input_ids=ids)      # hash-routed layers look tokens up by id
        use_ac = self.ac_every is not None and self.training and torch.is_grad_enabled()
        # recomputation re-runs everything but the attention kernel: its output (and lse) of the
        # first pass is kept, 2 bytes x q_dim per token and layer
        keep_attn = self.cache_attention and (self.ac_keep is None or "attention" in self.ac_keep)
        seq.attn_cache = {} if (use_ac and keep_attn) else None
        seq.op_stash = None
        if use_ac and self.ac_keep:
            from ..ops.stash import OpStash

            seq.op_stash = OpStash(self.ac_keep - {"attention"})
        for i, layer in enumerate(self.model.layers):
            if use_ac and i % self.ac_every == 0:
                h = checkpoint(self._run_layer, layer, i, h, seq, use_reentrant=False)
            else:
                h = self._run_layer(layer, i, h, seq)
        if self.arch.hc_mult:
            h = self.model.hc_head(h)
        return self.model.norm(h)

    def logprobs_entropy(self, hidden: torch.Tensor, labels: torch.Tensor,
                         inv_temperature: torch.Tensor | None = None, sampling_mask: torch.Tensor | None = None):
        """Per-token log-probability of ``labels`` and entropy, fp32 [T]. ``sampling_mask [T, K]``
        (ids the engine sampled from, -1 padded) renormalises the log-probabilities over those ids."""
        w = self.output_weight
        if self.lm_head is not None and self.lm_head.lora is not None:
            raise NotImplementedError("LoRA on lm_head is not supported with the fused head")
        labels = labels.reshape(-1)
        if self.arch.final_logit_softcapping:
            lp, ent = ops.softcapped_logprob_entropy(hidden, w, labels, inv_temperature,
                                                     self.arch.final_logit_softcapping)
        else:
            lp, ent = ops.fused_logprob_entropy(hidden, w, labels, inv_temperature)
        if sampling_mask is not None:
            if self.arch.final_logit_softcapping:
                raise NotImplementedError("sampling-mask replay with a soft-capped head")
            lp = ops.replay_sampling_mask(lp, hidden, w, labels, inv_temperature, sampling_mask)
        return lp, ent

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.output_weight)

    # ------------------------------------------------------------------ MoE helpers
    def moe_layers(self) -> Iterable[MoE]:
        for layer in self.model.layers:
            if isinstance(getattr(layer, "mlp", None), MoE):
                yield layer.mlp

    def load_balance_stats(self) -> dict[str, torch.Tensor]:
        """max-violation of the per-expert token share, averaged over MoE layers (the
        reference's ``max_vio`` metric)."""
        vios = []
        for m in self.moe_layers():
            if m.last_counts is None:
                continue
            c = m.last_counts.float()
            vios.append((c.max() - c.mean()) / c.mean().clamp_min(1.0))
        if not vios:
            return {}
        return {"max_vio": torch.stack(vios).mean()}


# ---------------------------------------------------------------------- LoRA / freezing
def _matches(name: str, patterns: list[str]) -> bool:
    parts = name.split(".")
    for pat in patterns:
        if pat in parts or re.search(pat, name):
            return True
    return False


_FUSED_MEMBERS = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}


def apply_fp8_training(model: CausalLM, ignore_patterns: list[str] | None = None, cache_weights: bool = True) -> list[str]:
    """Switches the projections (and expert stacks) whose name matches none of ``ignore_patterns`` (regular
    expressions, searched in the module name) to block-scaled fp8 for the forward product and the input gradient
    (``ops/fp8.py``); modules with an adapter, or with a dimension that is not a multiple of 16, keep bf16.
    Reference: src/prime_rl/trainer/models/layers/fp8_linear.py (module swap by name filter). Returns the names."""
    import re

    from ..ops import fp8 as fp8_ops

    fp8_ops.CACHE_WEIGHTS = cache_weights
    pats = [re.compile(p) for p in (ignore_patterns or [])]
    done: list[str] = []
    for name, mod in model.named_modules():
        if any(p.search(name) for p in pats):
            continue
        if isinstance(mod, Linear) and mod.lora is None and mod.weight.shape[0] % 16 == 0 and mod.weight.shape[1] % 16 == 0:
            mod.fp8_train = True
            done.append(name)
        elif isinstance(mod, GroupedExperts) and mod.lora_gate_up is None and mod.lora_down is None and \
                all(d % 16 == 0 for d in (*mod.gate_up_proj.shape[1:], *mod.down_proj.shape[1:])):
            mod.fp8_train = True
            done.append(name)
    return done


def check_context_parallel(arch, cp: int, cp_style: str) -> None:
    """Families with recurrent mixers split heads instead of the sequence around convolution and scan, which needs
    contiguous chunks per rank: ``cp_style = "ulysses"``."""
    recurrent = ("mamba" in (arch.block_types or [])) or ("gated_delta_net" in (arch.mixer_types or []))
    if cp > 1 and recurrent and cp_style != "ulysses":
        raise ValueError(f"model type '{arch.model_type}' has recurrent mixers: context parallelism needs "
                         f"model.cp_style = 'ulysses' (got '{cp_style}')")


def setup_quantization(model: CausalLM, mc, logger=None) -> list[str]:
    """``model.quantization`` of the trainer config: fp8 = block-scaled e4m3 (1 x 128 activation groups, 128 x 128
    weight blocks) for the forward products and input gradients of the projections outside ``ignore_patterns``. The
    MXFP8 recipes (UE8M0 scales over groups of 32) are not built."""
    q = mc.quantization
    if q is None:
        return []
    if q.type != "fp8":
        raise NotImplementedError(f"model.quantization.type = '{q.type}' is not built (block-scaled 'fp8' is)")
    names = apply_fp8_training(model, q.ignore_patterns, cache_weights=getattr(mc, "zero_stage", 2) != 3)
    from ..ops import fp8 as fp8_ops

    fp8_ops.FP8_WGRAD = getattr(q, "wgrad", "bf16") == "fp8"
    if logger is not None:
        logger.info(f"fp8 training: forward product and input gradient in block-scaled e4m3 on {len(names)} modules")
    return names


def apply_lora(model: CausalLM, rank: int, alpha: float, target_modules: list[str],
               modules_to_save: list[str] | None = None, seed: int = 0, num_adapters: int = 1) -> list[str]:
    """Freezes the base model and attaches adapters to every targeted projection. A fused
    projection gets one adapter segment per member that is targeted; members that are not
    targeted keep a zero-width contribution. ``num_adapters > 1``: every projection gets that many independent
    adapters (``layers.MultiLoRA``), chosen per token by ``layers.set_lora_num_tokens``. Returns the names of
    adapted modules."""
    arch = model.arch

    def many(make):
        return make() if num_adapters == 1 else MultiLoRA([make() for _ in range(num_adapters)])

    for p in model.parameters():
        p.requires_grad_(False)
    adapted: list[str] = []
    dtype = next(model.parameters()).dtype
    device = next(model.parameters()).device
    for name, mod in model.named_modules():
        leaf = name.split(".")[-1]
        if isinstance(mod, Linear) and leaf not in ("gate", "lm_head"):
            members = _FUSED_MEMBERS.get(leaf, [leaf])
            full = [name.rsplit(".", 1)[0] + "." + m if "." in name else m for m in members]
            if not all(_matches(f, target_modules) for f in full):
                if any(_matches(f, target_modules) for f in full):
                    raise ValueError(f"{name}: LoRA must target all of {members} or none (fused projection)")
                continue
            if leaf == "qkv_proj":
                segs = [mod.weight.shape[0] - 2 * arch.kv_dim, arch.kv_dim, arch.kv_dim]
            elif leaf == "gate_up_proj":
                half = mod.weight.shape[0] // 2
                segs = [half, half]
            else:
                segs = [mod.weight.shape[0]]
            mod.lora = many(lambda: LoRAAdapter(mod.weight.shape[1], segs, rank, alpha, members, dtype=dtype,
                                                device=device))
            adapted.append(name)
        elif isinstance(mod, GroupedExperts) and _matches(name, target_modules):
            E, width, H = mod.gate_up_proj.shape
            segs = [width // 2, width // 2] if width == 2 * arch.moe_intermediate_size else [width]
            mod.lora_gate_up = many(lambda: LoRAAdapter(H, segs, rank, alpha, ["gate_proj", "up_proj"][: len(segs)],
                                                        num_experts=E, dtype=dtype, device=device))
            mod.lora_down = many(lambda: LoRAAdapter(mod.down_proj.shape[2], [H], rank, alpha, ["down_proj"],
                                                     num_experts=E, dtype=dtype, device=device))
            adapted.append(name)
    # deterministic adapter init, identical on every data-parallel replica
    for i, (name, mod) in enumerate((n, m) for n, m in model.named_modules() if isinstance(m, LoRAAdapter)):
        mod.reset(seed=seed * 100003 + i)
    for name, p in model.named_parameters():
        if "lora_" in name or (modules_to_save and _matches(name, modules_to_save)):
            p.requires_grad_(True)
    return adapted


def freeze_router(model: CausalLM) -> None:
    for m in model.moe_layers():
        for p in m.router.parameters():
            p.requires_grad_(False)


def quantize_fp8_(model, skip: tuple[str, ...] = ("lm_head", "embed_tokens", "router", "g_proj"),
                  drop_bf16: bool = False) -> int:
    """Gives every eligible projection of ``model`` (dense linears and grouped experts) a
    block-scaled fp8 copy that no-grad forwards use instead of the bf16 weight (the rollout
    engine's ``weight_dtype = "fp8"``); call again after the bf16 weights changed. With
    ``drop_bf16`` the bf16 storage of the quantised projections is released. Returns the number of
    quantised modules."""
    n = 0
    for name, mod in model.named_modules():
        if any(s in name for s in skip) or not hasattr(mod, "quantize_fp8_"):
            continue
        n += bool(mod.quantize_fp8_(drop_bf16=drop_bf16))
    return n


def build_model(arch: ModelArch, *, device, dtype=torch.bfloat16, attn_backend: str = "auto", seed: int = 0,
                init: bool = True) -> CausalLM:
    model = CausalLM(arch, attn_backend=attn_backend, dtype=dtype, device=device)
    if init:
        model.init_weights(seed)
    return model
