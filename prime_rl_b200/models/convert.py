"""State-dict layouts and the invertible conversions between them.

Three layouts exist:

``native``  what the modules hold: fused ``self_attn.qkv_proj``, ``mlp.gate_up_proj``,
            ``mlp.experts.gate_up_proj [E, 2I, H]``.
``prime``   the checkpoint layout (DCP ``app.model.*``): per-projection names, experts stacked
            ``mlp.experts.{gate,up,down}_proj [E, ., .]``, router at ``mlp.router.gate.weight``
            (reference: trainer/models/qwen3_moe/modeling_qwen3_moe.py:43-224).
``hf``      HuggingFace names: ``mlp.gate.weight`` and one tensor per expert
            ``mlp.experts.{e}.{gate,up,down}_proj.weight``
            (reference: trainer/models/qwen3_moe/converting_qwen3_moe.py:8-14).

Conversions are built from small invertible ops (rename / split-concat / stack), in the
spirit of the reference's ``conversion_ops.py`` but written against plain dicts.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Callable

import torch

from .config import ModelArch

StateDict = dict[str, torch.Tensor]


# ---------------------------------------------------------------------- invertible ops
@dataclass
class Rename:
    """Regex rename; ``inverse`` swaps pattern and replacement templates."""

    pattern: str
    repl: str
    inv_pattern: str
    inv_repl: str

    def forward(self, sd: StateDict) -> StateDict:
        return {re.sub(self.pattern, self.repl, k): v for k, v in sd.items()}

    def inverse(self, sd: StateDict) -> StateDict:
        return {re.sub(self.inv_pattern, self.inv_repl, k): v for k, v in sd.items()}


@dataclass
class SplitConcat:
    """One fused tensor <-> several tensors concatenated on ``dim``; ``sizes(key_prefix)``
    gives the member widths."""

    fused_suffix: str
    member_suffixes: list[str]
    sizes: Callable[[torch.Tensor], list[int]]
    dim: int = 0

    def forward(self, sd: StateDict) -> StateDict:  # fused -> members
        out: StateDict = {}
        for k, v in sd.items():
            if k.endswith(self.fused_suffix):
                base = k[: -len(self.fused_suffix)]
                for suf, part in zip(self.member_suffixes, torch.split(v, self.sizes(v), dim=self.dim)):
                    out[base + suf] = part
            else:
                out[k] = v
        return out

    def inverse(self, sd: StateDict) -> StateDict:  # members -> fused
        out: StateDict = {}
        groups: dict[str, dict[str, torch.Tensor]] = {}
        for k, v in sd.items():
            for suf in self.member_suffixes:
                if k.endswith(suf):
                    groups.setdefault(k[: -len(suf)], {})[suf] = v
                    break
            else:
                out[k] = v
        for base, members in groups.items():
            if len(members) != len(self.member_suffixes):
                for suf, v in members.items():
                    out[base + suf] = v
                continue
            out[base + self.fused_suffix] = torch.cat([members[s] for s in self.member_suffixes], dim=self.dim)
        return out


@dataclass
class StackExperts:
    """Stacked ``[E, ...]`` tensor <-> one tensor per expert."""

    stacked_suffix: str      # e.g. "mlp.experts.gate_proj"
    per_expert_fmt: str      # e.g. "mlp.experts.{e}.gate_proj.weight"
    first: int = 0           # global index of the first stacked expert (expert-parallel ranks hold a range)

    def forward(self, sd: StateDict) -> StateDict:  # stacked -> per expert
        out: StateDict = {}
        for k, v in sd.items():
            if k.endswith(self.stacked_suffix):
                base = k[: -len(self.stacked_suffix)]
                for e in range(v.shape[0]):
                    out[base + self.per_expert_fmt.format(e=self.first + e)] = v[e]
            else:
                out[k] = v
        return out

    def inverse(self, sd: StateDict) -> StateDict:
        pat = re.compile("^(.*)" + re.escape(self.per_expert_fmt).replace(r"\{e\}", r"(\d+)") + "$")
        out: StateDict = {}
        groups: dict[str, dict[int, torch.Tensor]] = {}
        for k, v in sd.items():
            m = pat.match(k)
            if m:
                groups.setdefault(m.group(1), {})[int(m.group(2))] = v
            else:
                out[k] = v
        for base, items in groups.items():
            out[base + self.stacked_suffix] = torch.stack([items[e] for e in sorted(items)], dim=0)
        return out


@dataclass
class GptOssExperts:
    """GPT-OSS checkpoints keep every layer's experts fused and input-major: ``gate_up_proj [E, H, 2I]`` with
    gate and up columns interleaved (gate = even columns), ``down_proj [E, I, H]``, and biases alike; the prime
    layout has ``gate_proj / up_proj [E, I, H]``, ``down_proj [E, H, I]`` and separate bias tensors
    (reference: src/prime_rl/trainer/models/gpt_oss/converting_gpt_oss.py:8-44)."""

    def forward(self, sd: StateDict) -> StateDict:       # prime -> hf
        out: StateDict = {}
        for k, v in sd.items():
            if k.endswith("mlp.experts.gate_proj"):
                base = k[:-len("gate_proj")]
                up = sd[base + "up_proj"]
                fused = v.new_empty(v.shape[0], v.shape[2], 2 * v.shape[1])
                fused[..., ::2] = v.transpose(-2, -1)
                fused[..., 1::2] = up.transpose(-2, -1)
                out[base + "gate_up_proj"] = fused
            elif k.endswith("mlp.experts.gate_proj_bias"):
                base = k[:-len("gate_proj_bias")]
                up = sd[base + "up_proj_bias"]
                fused = v.new_empty(v.shape[0], 2 * v.shape[1])
                fused[..., ::2] = v
                fused[..., 1::2] = up
                out[base + "gate_up_proj_bias"] = fused
            elif k.endswith(("mlp.experts.up_proj", "mlp.experts.up_proj_bias")):
                continue
            elif k.endswith("mlp.experts.down_proj"):
                out[k] = v.transpose(-2, -1).contiguous()
            else:
                out[k] = v
        return out

    def inverse(self, sd: StateDict) -> StateDict:       # hf -> prime
        out: StateDict = {}
        for k, v in sd.items():
            if k.endswith("mlp.experts.gate_up_proj"):
                base = k[:-len("gate_up_proj")]
                out[base + "gate_proj"] = v[..., ::2].transpose(-2, -1).contiguous()
                out[base + "up_proj"] = v[..., 1::2].transpose(-2, -1).contiguous()
            elif k.endswith("mlp.experts.gate_up_proj_bias"):
                base = k[:-len("gate_up_proj_bias")]
                out[base + "gate_proj_bias"] = v[..., ::2].contiguous()
                out[base + "up_proj_bias"] = v[..., 1::2].contiguous()
            elif k.endswith("mlp.experts.down_proj"):
                out[k] = v.transpose(-2, -1).contiguous()
            else:
                out[k] = v
        return out


@dataclass
class MapValue:
    """Renames ``suffix`` -> ``new_suffix`` and maps the tensor (``fwd``) / back (``inv``)."""

    suffix: str
    new_suffix: str
    fwd: Callable[[torch.Tensor], torch.Tensor]
    inv: Callable[[torch.Tensor], torch.Tensor]

    def forward(self, sd: StateDict) -> StateDict:
        return {(k[: -len(self.suffix)] + self.new_suffix if k.endswith(self.suffix) else k):
                (self.fwd(v) if k.endswith(self.suffix) else v) for k, v in sd.items()}

    def inverse(self, sd: StateDict) -> StateDict:
        return {(k[: -len(self.new_suffix)] + self.suffix if k.endswith(self.new_suffix) else k):
                (self.inv(v) if k.endswith(self.new_suffix) else v) for k, v in sd.items()}


class ExactMap:
    """Key-for-key rename given as ``{prime name: published name}``."""

    def __init__(self, table: dict[str, str]):
        self.fwd = dict(table)
        self.inv = {v: k for k, v in table.items()}

    def forward(self, sd: StateDict) -> StateDict:
        return {self.fwd.get(k, k): v for k, v in sd.items()}

    def inverse(self, sd: StateDict) -> StateDict:
        return {self.inv.get(k, k): v for k, v in sd.items()}


class Chain:
    def __init__(self, ops: list):
        self.ops = ops

    def forward(self, sd: StateDict) -> StateDict:
        for op in self.ops:
            sd = op.forward(sd)
        return sd

    def inverse(self, sd: StateDict) -> StateDict:
        for op in reversed(self.ops):
            sd = op.inverse(sd)
        return sd


# ---------------------------------------------------------------------- layout chains
def _plain(a: str, b: str) -> Rename:
    """Literal suffix rename a <-> b."""
    return Rename(re.escape(a) + "$", b, re.escape(b) + "$", a)


def native_to_prime_chain(arch: ModelArch) -> Chain:
    kv = arch.kv_dim
    ops: list = []
    # depthwise convolutions are stored [C, K] here and [C, 1, K] in checkpoints; gated norms as modules
    ops += [MapValue("conv1d_weight", "conv1d.weight", lambda v: v.unsqueeze(1), lambda v: v.squeeze(1)),
            _plain("conv1d_bias", "conv1d.bias"),
            Rename(r"(mamba|self_attn)\.norm_weight$", r"\1.norm.weight", r"(mamba|self_attn)\.norm\.weight$",
                   r"\1.norm_weight")]
    if arch.hidden_act == "relu2":
        # non-gated MLPs: the "gate_up" tensor is just the up projection
        ops += [_plain("mlp.experts.gate_up_proj", "mlp.experts.up_proj"),
                _plain("shared_experts.gate_up_proj.weight", "shared_experts.up_proj.weight"),
                _plain("mlp.gate_up_proj.weight", "mlp.up_proj.weight")]
        return Chain(ops + [
            SplitConcat("self_attn.qkv_proj.weight", ["self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                                      "self_attn.v_proj.weight"], lambda v: [v.shape[0] - 2 * kv, kv, kv]),
            SplitConcat("self_attn.qkv_proj.bias", ["self_attn.q_proj.bias", "self_attn.k_proj.bias",
                                                    "self_attn.v_proj.bias"], lambda v: [v.shape[0] - 2 * kv, kv, kv])])
    if arch.model_type not in ("qwen3_5", "qwen3_5_moe"):      # their gated attention keeps q / k / v separate
        ops += [
            # the query width comes from the tensor: families with per-layer head counts differ by layer
            SplitConcat("self_attn.qkv_proj.weight", ["self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                                      "self_attn.v_proj.weight"], lambda v: [v.shape[0] - 2 * kv, kv, kv]),
            SplitConcat("self_attn.qkv_proj.bias", ["self_attn.q_proj.bias", "self_attn.k_proj.bias",
                                                    "self_attn.v_proj.bias"], lambda v: [v.shape[0] - 2 * kv, kv, kv]),
        ]
    ops += [
        SplitConcat("mlp.experts.gate_up_proj", ["mlp.experts.gate_proj", "mlp.experts.up_proj"],
                    lambda v: [v.shape[1] // 2, v.shape[1] // 2], dim=1),
        SplitConcat("mlp.experts.gate_up_proj_bias", ["mlp.experts.gate_proj_bias", "mlp.experts.up_proj_bias"],
                    lambda v: [v.shape[1] // 2, v.shape[1] // 2], dim=1),
        SplitConcat("shared_experts.gate_up_proj.weight", ["shared_experts.gate_proj.weight",
                                                           "shared_experts.up_proj.weight"],
                    lambda v: [v.shape[0] // 2, v.shape[0] // 2]),
        SplitConcat("mlp.gate_up_proj.weight", ["mlp.gate_proj.weight", "mlp.up_proj.weight"],
                    lambda v: [v.shape[0] // 2, v.shape[0] // 2]),
    ]
    return Chain(ops)


def _family_chain(arch: ModelArch) -> list:
    """Renames that depend on the kind of every layer (Nemotron-H, Qwen3.5)."""
    ops: list = []
    if arch.model_type == "nemotron_h":
        for i, kind in enumerate(arch.block_types or []):
            ours = {"mamba": "mamba", "attention": "self_attn", "mlp": "mlp", "moe": "mlp"}[kind]
            ops.append(Rename(rf"^model\.layers\.{i}\.{ours}\.", f"model.layers.{i}.mixer.",
                              rf"^model\.layers\.{i}\.mixer\.", f"model.layers.{i}.{ours}."))
        ops += [Rename(r"^model\.embed_tokens\.weight$", "model.embeddings.weight",
                       r"^model\.embeddings\.weight$", "model.embed_tokens.weight"),
                Rename(r"^model\.norm\.weight$", "model.norm_f.weight", r"^model\.norm_f\.weight$", "model.norm.weight"),
                Rename(r"^model\.", "backbone.", r"^backbone\.", "model.")]
    elif arch.model_type in ("qwen3_5", "qwen3_5_moe"):
        for i, kind in enumerate(arch.mixer_types or []):
            if kind == "gated_delta_net":
                ops.append(Rename(rf"^model\.layers\.{i}\.self_attn\.", f"model.layers.{i}.linear_attn.",
                                  rf"^model\.layers\.{i}\.linear_attn\.", f"model.layers.{i}.self_attn."))
        # zero-centred RMSNorm: checkpoints hold w - 1 (the gated norm inside linear_attn is a plain weight)
        for suf in ("input_layernorm.weight", "post_attention_layernorm.weight", "q_norm.weight", "k_norm.weight",
                    "model.norm.weight"):
            ops.append(MapValue(suf, suf, lambda v: v - 1, lambda v: v + 1))
    return ops


def _deepseek_v4_chain(arch: ModelArch, first_expert: int = 0) -> Chain:
    """The published DeepSeek-V4 checkpoints use a compact naming without a ``model.`` prefix
    (``layers.N.attn.wq_a``, ``ffn.experts.E.w1`` ...; reference:
    src/prime_rl/trainer/models/deepseek_v4/converting_deepseek_v4.py:27-106)."""
    table = {"model.embed_tokens.weight": "embed.weight", "model.norm.weight": "norm.weight",
             "lm_head.weight": "head.weight", "model.hc_head.hc_fn": "hc_head_fn",
             "model.hc_head.hc_base": "hc_head_base", "model.hc_head.hc_scale": "hc_head_scale"}
    comp = {"kv_proj.weight": "wkv.weight", "gate_proj.weight": "wgate.weight", "kv_norm.weight": "norm.weight",
            "position_bias": "ape"}
    for i in range(arch.num_hidden_layers):
        a = b = f"model.layers.{i}"          # the last op of the chain strips the `model.` prefix of the layers
        table.update({f"{a}.input_layernorm.weight": f"{b}.attn_norm.weight",
                      f"{a}.post_attention_layernorm.weight": f"{b}.ffn_norm.weight"})
        for hc, short in (("attn_hc", "hc_attn"), ("ffn_hc", "hc_ffn")):
            for leaf in ("fn", "base", "scale"):
                table[f"{a}.{hc}.{leaf}"] = f"{b}.{short}_{leaf}"
        for ours, theirs in (("q_a_proj.weight", "wq_a.weight"), ("q_a_norm.weight", "q_norm.weight"),
                             ("q_b_proj.weight", "wq_b.weight"), ("kv_proj.weight", "wkv.weight"),
                             ("kv_norm.weight", "kv_norm.weight"), ("o_a_proj.weight", "wo_a.weight"),
                             ("o_b_proj.weight", "wo_b.weight"), ("sinks", "attn_sink")):
            table[f"{a}.self_attn.{ours}"] = f"{b}.attn.{theirs}"
        for ours, theirs in comp.items():
            table[f"{a}.self_attn.compressor.{ours}"] = f"{b}.attn.compressor.{theirs}"
            table[f"{a}.self_attn.indexer.compressor.{ours}"] = f"{b}.attn.indexer.compressor.{theirs}"
        table[f"{a}.self_attn.indexer.q_b_proj.weight"] = f"{b}.attn.indexer.wq_b.weight"
        table[f"{a}.self_attn.indexer.weights_proj.weight"] = f"{b}.attn.indexer.weights_proj.weight"
        table.update({f"{a}.mlp.router.gate.weight": f"{b}.ffn.gate.weight",
                      f"{a}.mlp.router.e_score_correction_bias": f"{b}.ffn.gate.bias",
                      f"{a}.mlp.router.tid2eid": f"{b}.ffn.gate.tid2eid",
                      f"{a}.mlp.shared_experts.gate_proj.weight": f"{b}.ffn.shared_experts.w1.weight",
                      f"{a}.mlp.shared_experts.down_proj.weight": f"{b}.ffn.shared_experts.w2.weight",
                      f"{a}.mlp.shared_experts.up_proj.weight": f"{b}.ffn.shared_experts.w3.weight"})
    return Chain([StackExperts("mlp.experts.gate_proj", "ffn.experts.{e}.w1.weight", first_expert),
                  StackExperts("mlp.experts.down_proj", "ffn.experts.{e}.w2.weight", first_expert),
                  StackExperts("mlp.experts.up_proj", "ffn.experts.{e}.w3.weight", first_expert),
                  ExactMap(table),
                  Rename(r"^model\.layers\.", "layers.", r"^layers\.", "model.layers.")])


def prime_to_hf_chain(arch: ModelArch, first_expert: int = 0) -> Chain:
    """``first_expert``: global index of the first expert in the stacked tensors (an expert-parallel
    rank exports its own range under global numbers)."""
    if arch.model_type == "deepseek_v4":
        return _deepseek_v4_chain(arch, first_expert)
    ops: list = []
    if arch.model_type in ("qwen3_5_moe",):
        ops += [Rename(r"mlp\.shared_experts\.", r"mlp.shared_expert.", r"mlp\.shared_expert\.", r"mlp.shared_experts.")]
    if arch.model_type == "nemotron_h" and arch.is_moe:
        ops += [Rename(r"mlp\.router\.gate\.(weight|bias)$", r"mlp.gate.\1", r"mlp\.gate\.(weight|bias)$",
                       r"mlp.router.gate.\1"),
                Rename(r"mlp\.router\.e_score_correction_bias$", r"mlp.gate.e_score_correction_bias",
                       r"mlp\.gate\.e_score_correction_bias$", r"mlp.router.e_score_correction_bias"),
                StackExperts("mlp.experts.up_proj", "mlp.experts.{e}.up_proj.weight", first_expert),
                StackExperts("mlp.experts.down_proj", "mlp.experts.{e}.down_proj.weight", first_expert)]
        return Chain(ops + _family_chain(arch))
    if arch.model_type == "gpt_oss":
        return Chain([Rename(r"mlp\.router\.gate\.(weight|bias)$", r"mlp.router.\1", r"mlp\.router\.(weight|bias)$",
                             r"mlp.router.gate.\1"), GptOssExperts()])
    if arch.model_type == "laguna":
        # Laguna checkpoints name the shared expert in the singular and keep the selection bias under `experts`
        ops += [
            Rename(r"mlp\.shared_experts\.", r"mlp.shared_expert.", r"mlp\.shared_expert\.", r"mlp.shared_experts."),
            Rename(r"mlp\.router\.e_score_correction_bias$", r"mlp.experts.e_score_correction_bias",
                   r"mlp\.experts\.e_score_correction_bias$", r"mlp.router.e_score_correction_bias"),
        ]
    if arch.is_moe:
        ops += [
            Rename(r"mlp\.router\.gate\.(weight|bias)$", r"mlp.gate.\1", r"mlp\.gate\.(weight|bias)$",
                   r"mlp.router.gate.\1"),
            Rename(r"mlp\.router\.e_score_correction_bias$", r"mlp.gate.e_score_correction_bias",
                   r"mlp\.gate\.e_score_correction_bias$", r"mlp.router.e_score_correction_bias"),
            StackExperts("mlp.experts.gate_proj", "mlp.experts.{e}.gate_proj.weight", first_expert),
            StackExperts("mlp.experts.up_proj", "mlp.experts.{e}.up_proj.weight", first_expert),
            StackExperts("mlp.experts.down_proj", "mlp.experts.{e}.down_proj.weight", first_expert),
        ]
    return Chain(ops + _family_chain(arch))


def native_to_prime(sd: StateDict, arch: ModelArch) -> StateDict:
    return native_to_prime_chain(arch).forward(sd)


def prime_to_native(sd: StateDict, arch: ModelArch) -> StateDict:
    return native_to_prime_chain(arch).inverse(sd)


def prime_to_hf(sd: StateDict, arch: ModelArch, first_expert: int = 0) -> StateDict:
    sd = prime_to_hf_chain(arch, first_expert).forward(sd)
    if arch.tie_word_embeddings:
        sd.pop("lm_head.weight", None)
    return sd


def hf_to_prime(sd: StateDict, arch: ModelArch) -> StateDict:
    return prime_to_hf_chain(arch).inverse(sd)


def native_to_hf(sd: StateDict, arch: ModelArch) -> StateDict:
    return prime_to_hf(native_to_prime(sd, arch), arch)


def hf_to_native(sd: StateDict, arch: ModelArch) -> StateDict:
    return prime_to_native(hf_to_prime(sd, arch), arch)


def is_expert_sharded_key(key: str) -> bool:
    """Tensors that expert parallelism slices on their leading (expert) dimension, in the native and
    prime layouts: the stacked expert projections and the adapters attached to them."""
    return ".mlp.experts." in key and not key.endswith("e_score_correction_bias")


def expert_parallel_info(model):
    """``None`` or the record ``install_expert_parallel`` leaves on the model: ``ep``, ``ep_rank``,
    ``group`` (the ep process group), ``num_experts``, ``local_experts``, ``writer`` (this rank's ep
    group is the one that exports weights when several groups replicate the experts)."""
    info = getattr(model, "ep_info", None)
    return info if info is not None and info["ep"] > 1 else None


def model_state(model, layout: str = "prime", include_lora: bool = False, gather_experts: bool = False) -> StateDict:
    """State dict of a CausalLM in the requested layout (views, no copies where possible).

    With expert parallelism every rank holds ``[E / ep, ...]`` slices: ``layout="hf"`` then numbers
    this rank's experts globally; ``gather_experts=True`` (a collective over the ep group, every
    rank of it must call) returns the full stacks instead."""
    sd = {k: v for k, v in model.state_dict().items() if include_lora or "lora_" not in k}
    info = expert_parallel_info(model)
    first = 0
    if info is not None:
        if gather_experts:
            sd = {k: (gather_expert_shards(v, info) if is_expert_sharded_key(k) else v) for k, v in sd.items()}
        else:
            first = info["ep_rank"] * info["local_experts"]
    if layout == "native":
        return sd
    sd = native_to_prime(sd, model.arch)
    return sd if layout == "prime" else prime_to_hf(sd, model.arch, first)


def gather_expert_shards(local: torch.Tensor, info) -> torch.Tensor:
    """All-gather of one expert-sharded tensor over the ep group -> ``[E, ...]`` on every rank."""
    import torch.distributed as dist

    parts = [torch.empty_like(local) for _ in range(info["ep"])]
    dist.all_gather(parts, local.detach().contiguous(), group=info["group"])
    return torch.cat(parts, dim=0)


@torch.no_grad()
def load_model_state(model, sd: StateDict, layout: str = "prime", strict: bool = True) -> None:
    arch = model.arch
    if arch.tie_word_embeddings and layout in ("hf", "prime") and "lm_head.weight" in sd:
        sd = {k: v for k, v in sd.items() if k != "lm_head.weight"}      # the tied head is the embedding
    if layout == "hf":
        sd = hf_to_prime(sd, arch)
    if layout in ("hf", "prime"):
        sd = prime_to_native(sd, arch)
    own = model.state_dict()
    missing = [k for k in own if k not in sd and "lora_" not in k and not k.endswith("inv_freq")]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"state dict mismatch: missing={missing[:5]} unexpected={unexpected[:5]}")
    shard = getattr(model, "tp_shard", None)      # engine tensor parallelism: this process keeps one slice
    info = expert_parallel_info(model)
    for k, v in sd.items():
        if k in own:
            if info is not None and is_expert_sharded_key(k) and v.shape[0] == info["num_experts"] != own[k].shape[0]:
                lo = info["ep_rank"] * info["local_experts"]      # a full stack: keep this rank's expert range
                v = v[lo:lo + info["local_experts"]]
            v = v if shard is None else shard(k, v)
            if own[k].numel() == 0 and v.numel() > 0:
                # a serving model that released the bf16 storage of its fp8 projections: quantise the new
                # values straight into the fp8 copy
                owner_name, leaf = k.rsplit(".", 1)
                owner = model.get_submodule(owner_name)
                src = v.to(own[k].device)
                ok = owner.quantize_fp8_(drop_bf16=True, source={leaf: src} if hasattr(owner, "gate_up_proj") else src)
                if not ok:
                    raise RuntimeError(f"{k}: the bf16 storage was released but the module cannot be re-quantised")
                continue
            own[k].copy_(v.to(own[k].dtype))


# ---------------------------------------------------------------------- LoRA adapters (PEFT layout)
def lora_to_peft(model) -> StateDict:
    """Adapter tensors under PEFT names ``base_model.model.<module>.lora_{A,B}.weight``; fused
    projections are split back into their members; experts keep a leading ``[E]`` dim."""
    out: StateDict = {}
    from .layers import LoRAAdapter

    for name, mod in model.named_modules():
        if not isinstance(mod, LoRAAdapter):
            continue
        owner = name.rsplit(".", 1)[0]                      # module that holds the adapter
        parent = owner.rsplit(".", 1)[0] if "." in owner else ""
        is_expert = name.endswith("lora_gate_up") or name.endswith("lora_down")
        r = mod.rank
        for s, member in enumerate(mod.names):
            a = mod.lora_A[..., s * r:(s + 1) * r, :]
            b = mod.lora_B[s]
            target = f"{owner}.{member}" if is_expert else f"{parent}.{member}"
            out[f"base_model.model.{target}.lora_A.weight"] = a.detach()
            out[f"base_model.model.{target}.lora_B.weight"] = b.detach()
    return out
