"""Trainer configuration (field names follow the reference's ``configs/trainer.py``)."""

from __future__ import annotations

import warnings
from pathlib import Path
from typing import Annotated, Any, Literal, TypeAlias

from pydantic import BeforeValidator, Field, model_validator

from .base import BaseConfig
from .monitors import MonitorsConfig
from .shared import (BaseModelConfig, BaseWeightBroadcastConfig, EnvVars, FileSystemTransportConfig,  # noqa: F401
                     HeartbeatConfig, MetricsServerConfig, ResumeConfig, TrainerLogConfig, TransportConfig,
                     ZMQTransportConfig, default_output_dir)

AttnImplementation: TypeAlias = Literal["auto", "sdpa", "eager", "flash_attention_2", "flash_attention_3",
                                        "flash_attention_4", "tcgen05"]


class GCConfig(BaseConfig):
    interval: int = Field(50, ge=1)


class ActivationCheckpointConfig(BaseConfig):
    mode: Literal["full", "selective"] = "full"
    freq: int = Field(1, ge=1)
    targets: list[str] | None = None


class ActivationOffloadingConfig(BaseConfig):
    pin_memory: bool = True
    max_inflight_activations: int = Field(5, ge=1)


class OptimizerInBackwardOffloadConfig(BaseConfig):
    chunk_elements: int = Field(16 * 1024 * 1024, ge=1024)
    max_pinned_slots: int | None = Field(None, ge=1)
    cpu_optimizer_backend: Literal["native", "torch"] = "native"
    numa_bind: bool = True


def _normalize_full_offload(value):
    """``full_offload = true`` enables the block with its defaults, ``false`` disables it."""
    if value is True:
        return {}
    if value is False:
        return None
    return value


OptimizerInBackwardOffload: TypeAlias = Annotated[OptimizerInBackwardOffloadConfig | None,
                                                  BeforeValidator(_normalize_full_offload)]


class CompileConfig(BaseConfig):
    """Kept for config compatibility: the hot path here is hand-written kernels plus CUDA
    graphs, so this block only toggles graph capture of the per-layer launch sequence."""

    fullgraph: bool = False


class FusionsConfig(BaseConfig):
    enabled: list[Literal["gate_up", "qkv"]] = ["gate_up", "qkv"]
    raise_on_fail: bool = False


class IndexCacheConfig(BaseConfig):
    topk_freq: int = Field(1, ge=1)
    topk_pattern: str | None = None


class LoRAConfig(BaseConfig):
    rank: int = Field(16, ge=1)
    alpha: float = Field(32.0, ge=0)
    dropout: float = Field(0.0, ge=0, le=1)
    target_modules: list[str] = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj",
                                 "experts", "fc1_latent_proj", "fc2_latent_proj"]
    modules_to_save: list[str] = []
    num_adapters: int = Field(1, ge=1)      # > 1: independent adapters chosen per token by ``lora_num_tokens``


class DebugModelConfig(BaseConfig):
    num_layers: int | None = None
    random_init: bool = False
    force_balanced_routing: bool = False


MXFP8Recipe: TypeAlias = Literal["mxfp8_rceil", "mxfp8_rceil_wgrad_with_hp"]

_DEFAULT_FP8_IGNORE = ["lm_head", "router", r"mlp\.gate\.", r"shared_expert\.output_gate", "eh_proj", "weights_proj",
                       "in_proj_a", "in_proj_b"]


class FP8Config(BaseConfig):
    type: Literal["fp8"] = "fp8"
    ignore_patterns: list[str] = _DEFAULT_FP8_IGNORE
    # weight gradient of the dense projections: "bf16" product into the fp32 accumulator (default), or "fp8": dY^T in
    # 1 x 128 groups along the tokens times X^T in 128 x 128 blocks on the fp8 kernel, then added to the accumulator
    wgrad: Literal["bf16", "fp8"] = "bf16"


class MXFP8Config(BaseConfig):
    type: Literal["mxfp8"] = "mxfp8"
    recipe: MXFP8Recipe = "mxfp8_rceil"
    ignore_patterns: list[str] = _DEFAULT_FP8_IGNORE


QuantizationConfig: TypeAlias = Annotated[FP8Config | MXFP8Config, Field(discriminator="type")]


class MoEComputeConfigBase(BaseConfig):
    apply_to: str | list[Annotated[int, Field(ge=0, strict=True)]] = "all"

    def layers(self, num_layers: int) -> set[int]:
        """Layer indices this block applies to: "all", an explicit list, or "a-b,c" ranges."""
        if self.apply_to == "all":
            return set(range(num_layers))
        if isinstance(self.apply_to, list):
            return set(self.apply_to)
        out: set[int] = set()
        for part in str(self.apply_to).split(","):
            part = part.strip()
            if "-" in part:
                a, b = part.split("-")
                out.update(range(int(a), int(b) + 1))
            elif part:
                out.add(int(part))
        return out


class BF16MoEComputeConfig(MoEComputeConfigBase):
    type: Literal["bf16"] = "bf16"


class DeepGemmFP8MoEComputeConfig(MoEComputeConfigBase):
    """Block-scaled fp8 expert GEMMs (128x128 weight blocks, 1x128 activation scales)."""

    type: Literal["deepgemm_fp8"] = "deepgemm_fp8"


class MXFP8MoEComputeConfig(MoEComputeConfigBase):
    type: Literal["mxfp8"] = "mxfp8"
    recipe: MXFP8Recipe = "mxfp8_rceil"


MoEComputeConfig: TypeAlias = Annotated[
    BF16MoEComputeConfig | DeepGemmFP8MoEComputeConfig | MXFP8MoEComputeConfig, Field(discriminator="type")]


class TorchMoEDispatchConfig(BaseConfig):
    """Library all-to-all (NCCL / gloo) token dispatch: the baseline."""

    type: Literal["torch"] = "torch"
    transport: Literal["bf16", "mxfp8"] = "bf16"


class DeepEPMoEDispatchConfig(BaseConfig):
    """Kept for config compatibility; maps onto the peer-memory dispatcher."""

    type: Literal["deepep"] = "deepep"
    num_sms: int = Field(20, ge=1)
    token_chunk_size: int | None = Field(None, ge=1)


class P2PMoEDispatchConfig(BaseConfig):
    """Peer-memory (NVLink) dispatch/combine written by the routing kernels themselves."""

    type: Literal["p2p"] = "p2p"
    num_sms: int = Field(32, ge=1)
    # receive-buffer rows as a multiple of the rows a rank sends. None = the worst case (every token of every rank
    # routed to one rank: factor = ep), which cannot overflow however skewed the router is; a smaller factor saves
    # 4 buffers x rows x hidden x 2 bytes of memory and reports an overflow through the kernel status word
    capacity_factor: float | None = Field(None, gt=0)
    payload: Literal["bf16", "fp8"] = "bf16"    # fp8: e4m3 + 1x128 fp32 scales on the forward dispatch
    # forward dispatch without a global wait: rows leave on a side stream and the first expert GEMM's loader waits
    # per 128-row block. Measured a little slower than one wait at 2 and 8 GPUs (3.69 / 4.34 ms against 3.65 /
    # 4.25 ms per layer), hence off
    per_block_arrival: bool = False


MoEDispatchConfig: TypeAlias = Annotated[
    TorchMoEDispatchConfig | DeepEPMoEDispatchConfig | P2PMoEDispatchConfig, Field(discriminator="type")]


class MoERuntimeConfig(BaseConfig):
    compute: MoEComputeConfig = BF16MoEComputeConfig()
    dispatch: MoEDispatchConfig = TorchMoEDispatchConfig()


class ModelConfig(BaseModelConfig):
    conversion_dir: Path | None = None
    seq_len: int = 2048
    attn: AttnImplementation = "auto"
    compile: CompileConfig | None = CompileConfig()
    fusions: FusionsConfig = FusionsConfig()
    ac: ActivationCheckpointConfig | None = ActivationCheckpointConfig()
    ac_offloading: ActivationOffloadingConfig | None = None
    fsdp_cpu_offload: bool = False
    optim_cpu_offload: bool = False
    full_offload: OptimizerInBackwardOffload = None
    reshard_after_forward: bool = True
    dp_replicate: int = 1
    ep: int | Literal["auto"] = "auto"
    moe: MoERuntimeConfig = MoERuntimeConfig()
    cp: int = 1
    cp_style: Literal["ring", "ulysses"] = "ring"
    # K / V exchange of the ring style. "nccl": all-gather, then one attention call per query slice. "p2p": the forward
    # all-gather runs inside the attention kernel over NVLink peer memory. "ring": K / V blocks travel rank to rank,
    # one partial attention per step merged through the log-sum-exp, dK / dV partials returned to the owners (K / V of
    # the whole sequence never exist on one rank). "ring_p2p": the same ring with every block pulled straight from its
    # owner's symmetric memory on a side stream and the dK / dV partials summed by peer loads (one NVSwitch box).
    cp_kv_exchange: Literal["nccl", "p2p", "ring", "ring_p2p"] = "nccl"
    # "p2p": the sharded optimizer's gradient reduce-scatter (with cast / scale) and parameter all-gather run as
    # peer-memory kernels over NVLink instead of NCCL collectives (one NVSwitch box, at most 8 ranks per shard group)
    optim_collectives: Literal["nccl", "p2p"] = "nccl"
    # 2: bf16 parameters replicated, optimizer state (fp32 master, moments) and the gradient reduction partitioned
    # over the sharding ranks: one reduce-scatter and one all-gather per step. 3: parameters partitioned too (FSDP):
    # each decoder layer is all-gathered right before it runs (prefetched one layer ahead), re-gathered for its
    # recomputation in the backward pass, and its gradients are reduce-scattered as soon as they are complete.
    zero_stage: Literal[2, 3] = 2
    impl: Literal["hf", "custom", "auto"] = "auto"
    optimization_dtype: Literal["bfloat16", "float32"] = "float32"
    reduce_dtype: Literal["bfloat16", "float32"] = "float32"
    moe_router_dtype: Literal["bfloat16", "float32"] = "float32"
    quantization: QuantizationConfig | None = None
    index_cache: IndexCacheConfig | None = None
    freeze_moe_router: bool = False
    lora: LoRAConfig | None = None
    debug: DebugModelConfig = DebugModelConfig()
    fused_lm_head_token_chunk_size: int | Literal["disabled"] = 8192
    # architecture given inline instead of a HF config directory (random-init runs, benchmarks)
    arch: dict[str, Any] | None = None

    @model_validator(mode="after")
    def _checks(self):
        if self.trust_remote_code and self.impl not in ("hf", "auto"):
            raise ValueError("trust_remote_code needs model.impl = 'hf' or 'auto'")
        if self.vlm is not None and self.impl != "custom":
            raise ValueError("VLM training requires model.impl='custom'")
        if self.vlm is not None and self.cp > 1 and self.cp_style != "ulysses":
            raise ValueError("VLM models require cp_style='ulysses' for context parallelism")
        if self.cp > 1 and self.attn in ("sdpa", "eager"):
            raise ValueError("context parallelism needs a flash-attention implementation")
        if self.cp > 1 and self.impl not in ("custom", "auto"):
            raise ValueError("context parallelism requires model.impl='custom' or 'auto'")
        if self.ac_offloading is not None and self.ac is None:
            self.ac = ActivationCheckpointConfig()
        if self.fsdp_cpu_offload and (self.optim_cpu_offload or self.full_offload):
            raise ValueError("fsdp_cpu_offload cannot be combined with optimizer CPU offloading")
        if self.optim_cpu_offload and self.full_offload:
            raise ValueError("optim_cpu_offload and full_offload are mutually exclusive")
        if self.quantization is not None and self.impl not in ("custom", "auto"):
            raise ValueError(f"{self.quantization.type} training needs model.impl='custom' or 'auto'")
        if self.ep != 1:
            compute, dispatch = self.moe.compute, self.moe.dispatch
            if isinstance(dispatch, DeepEPMoEDispatchConfig) and isinstance(compute, MXFP8MoEComputeConfig):
                raise ValueError("MXFP8 expert compute does not support DeepEP dispatch")
            if isinstance(dispatch, TorchMoEDispatchConfig) and dispatch.transport == "mxfp8" \
                    and not isinstance(compute, MXFP8MoEComputeConfig):
                raise ValueError("MXFP8 transport requires model.moe.compute.type='mxfp8'")
        return self


class TokenizerConfig(BaseConfig):
    name: str | None = None
    trust_remote_code: bool | None = None
    chat_template: str | None = None


class ConstantSchedulerConfig(BaseConfig):
    type: Literal["constant"] = "constant"


class LinearSchedulerConfig(BaseConfig):
    type: Literal["linear"] = "linear"
    warmup_steps: int = Field(10, ge=0)
    decay_steps: int = Field(10, ge=0)
    min_lr: float = Field(0.0, ge=0)


class CosineSchedulerConfig(BaseConfig):
    type: Literal["cosine"] = "cosine"
    warmup_steps: int = Field(10, ge=0)
    min_lr: float = Field(0.0, ge=0)


SchedulerConfig: TypeAlias = Annotated[
    ConstantSchedulerConfig | LinearSchedulerConfig | CosineSchedulerConfig, Field(discriminator="type")]


def validate_scheduler(scheduler, max_steps: int | None) -> None:
    if isinstance(scheduler, LinearSchedulerConfig):
        if scheduler.warmup_steps == 0 and scheduler.decay_steps == 0:
            raise ValueError("linear scheduler needs warmup_steps > 0 or decay_steps > 0")
        if scheduler.decay_steps > 0:
            if max_steps is None:
                raise ValueError("max_steps is required for a linear scheduler with decay_steps > 0")
            if scheduler.warmup_steps + scheduler.decay_steps > max_steps:
                raise ValueError("warmup_steps + decay_steps must not exceed max_steps")
    if isinstance(scheduler, CosineSchedulerConfig):
        if max_steps is None:
            raise ValueError("max_steps is required for a cosine scheduler")
        if scheduler.warmup_steps >= max_steps:
            raise ValueError("warmup_steps must be less than max_steps")


class BaseOptimizerConfig(BaseConfig):
    lr: float = Field(1e-6, ge=0)
    weight_decay: float = Field(0.01, ge=0)
    max_norm: float | None = Field(1.0, ge=0)


class SGDConfig(BaseOptimizerConfig):
    type: Literal["sgd"] = "sgd"
    nesterov: bool = True
    momentum: float = 0.9


class AdamWConfig(BaseOptimizerConfig):
    type: Literal["adamw"] = "adamw"
    betas1: float = 0.9
    betas2: float = 0.999
    eps: float = 1e-8


class MuonConfig(BaseOptimizerConfig):
    type: Literal["muon"] = "muon"
    mu: float = Field(0.95, ge=0)
    betas1: float = 0.9
    betas2: float = 0.999
    ns_steps: int = 5
    adjust_lr: Literal["spectral_norm", "rms_norm"] | None = "rms_norm"
    # every matrix is orthogonalised by ONE data-parallel rank (matrices dealt out by cost), the updates are summed
    # over the ranks afterwards; False: every rank orthogonalises every matrix
    distributed: bool = True


class SignSGDConfig(BaseOptimizerConfig):
    type: Literal["sign_sgd"] = "sign_sgd"


OptimizerConfig: TypeAlias = Annotated[SGDConfig | AdamWConfig | MuonConfig | SignSGDConfig,
                                       Field(discriminator="type")]


class CheckpointConfig(BaseConfig):
    output_dir: Path | None = None
    interval: int | None = Field(None, ge=1)
    keep_last: int | None = Field(None, ge=1)
    keep_interval: int | None = Field(None, ge=1)
    skip_progress: bool = False
    skip_scheduler: bool = False
    skip_dataloader: bool = False
    skip_optimizer: bool = False


class IPOLossConfig(BaseConfig):
    type: Literal["ipo"] = "ipo"
    eps: float = Field(0.1, ge=0)
    adv_tau: float = Field(1.0, ge=0)
    kl_tau: float = Field(1e-3, ge=0)


class IcePopLossConfig(BaseConfig):
    type: Literal["icepop"] = "icepop"
    ratio_low: float = Field(0.2, gt=0)
    ratio_high: float = Field(5.0, gt=0)
    adv_tau: float = Field(1.0, ge=0)

    @model_validator(mode="after")
    def _band(self):
        if self.ratio_low >= self.ratio_high:
            raise ValueError("ratio_low must be below ratio_high")
        return self


class CustomLossConfig(BaseConfig):
    type: Literal["custom"] = "custom"
    import_path: str
    kwargs: dict[str, Any] = Field(default_factory=dict)


LossConfig: TypeAlias = Annotated[IPOLossConfig | IcePopLossConfig | CustomLossConfig, Field(discriminator="type")]


class FakeDataLoaderConfig(BaseConfig):
    batch_size: int = Field(2, ge=1)
    generate_samples: bool = False


class DataLoaderConfig(BaseConfig):
    fake: FakeDataLoaderConfig | None = None


class FileSystemWeightBroadcastConfig(BaseWeightBroadcastConfig):
    type: Literal["filesystem"] = "filesystem"


class InMemoryWeightBroadcastConfig(BaseWeightBroadcastConfig):
    host: str = "localhost"
    port: int
    inference_world_size: int = 1


class NCCLWeightBroadcastConfig(InMemoryWeightBroadcastConfig):
    type: Literal["nccl"] = "nccl"
    port: int = 29501
    quantize_in_weight_transfer: bool = False


class NIXLWeightBroadcastConfig(InMemoryWeightBroadcastConfig):
    type: Literal["nixl"] = "nixl"
    port: int = 8001
    session_id: str = "default"
    overlap_transfer_and_replay: bool = False


class P2PWeightBroadcastConfig(InMemoryWeightBroadcastConfig):
    """Trainer shards are pushed into the engine's buffers over NVLink peer memory by a
    kernel that quantises to block-scaled fp8 on the way (same box only)."""

    type: Literal["p2p"] = "p2p"
    port: int = 29502
    quantize_in_weight_transfer: bool = True


WeightBroadcastConfig: TypeAlias = Annotated[
    FileSystemWeightBroadcastConfig | NCCLWeightBroadcastConfig | NIXLWeightBroadcastConfig
    | P2PWeightBroadcastConfig, Field(discriminator="type")]


class TrainerConfig(BaseConfig):
    model: ModelConfig = ModelConfig()
    tokenizer: TokenizerConfig = TokenizerConfig()
    data: DataLoaderConfig = DataLoaderConfig()
    loss: LossConfig = IPOLossConfig()
    optim: OptimizerConfig = AdamWConfig()
    scheduler: SchedulerConfig = ConstantSchedulerConfig()
    ckpt: CheckpointConfig | None = None
    resume: ResumeConfig | None = None
    weight_broadcast: WeightBroadcastConfig = FileSystemWeightBroadcastConfig()
    rollout_transport: TransportConfig = ZMQTransportConfig()
    log: TrainerLogConfig = TrainerLogConfig()
    monitors: MonitorsConfig = MonitorsConfig()
    output_dir: Path = Field(default_factory=default_output_dir)
    matmul_precision: Literal["highest", "high", "medium"] = "high"
    max_steps: int | None = None
    enable_router_replay: bool = False
    log_annotations: bool = False          # per-token trainer logprob / entropy of traced rollouts -> monitors
    memory_profiler_path: Path | None = None
    gc: GCConfig | None = GCConfig()
    trace_path: Path | None = None
    dist_timeout_seconds: int = 3600
    heartbeat: HeartbeatConfig | None = None
    metrics_server: MetricsServerConfig | None = None
    env_vars: EnvVars = {}
    max_concurrent_runs: int = 1
    dry_run: bool = False

    @model_validator(mode="after")
    def _checks(self):
        if self.model.ep != 1 and self.model.moe.dispatch.type == "deepep" and self.optim.max_norm is not None:
            warnings.warn("gradient clipping is not compatible with DeepEP-style dispatch; disabling max_norm",
                          stacklevel=1)
            self.optim.max_norm = None
        if self.model.full_offload and self.optim.type not in ("adamw", "sign_sgd"):
            raise ValueError("full optimizer offload only supports AdamW and SignSGD")
        if self.model.full_offload and self.optim.max_norm is not None:
            warnings.warn("gradient clipping prevents optimizer-in-backward overlap; disabling max_norm",
                          stacklevel=1)
            self.optim.max_norm = None
        if self.model.vlm is not None and not self.model.vlm.freeze_vision_encoder and self.model.lora is not None:
            raise ValueError("freeze_vision_encoder=false is incompatible with LoRA")
        if self.trace_path:
            if self.max_steps is None:
                raise ValueError("max_steps is required when tracing")
            if self.max_steps >= 10:
                raise ValueError("tracing 10 or more steps produces traces too large to load")
        validate_scheduler(self.scheduler, self.max_steps)
        if self.optim.type == "muon" and self.model.fsdp_cpu_offload:
            raise ValueError("Muon does not support FSDP CPU offload")
        if self.model.lora is not None and self.weight_broadcast.type in ("nccl", "nixl", "p2p"):
            raise ValueError("LoRA requires weight_broadcast.type = 'filesystem' (adapters are loaded from disk)")
        if self.model.lora is not None and self.model.lora.modules_to_save and self.data.fake is None:
            raise ValueError("model.lora.modules_to_save cannot be served by the adapter broadcast")
        if self.tokenizer.name is None:
            self.tokenizer.name = self.model.name
        if self.tokenizer.trust_remote_code is None:
            self.tokenizer.trust_remote_code = self.model.trust_remote_code
        if self.model.ep not in (1, "auto") and self.model.impl not in ("custom", "auto"):
            raise ValueError("EP is only supported with the custom implementation or auto mode")
        if self.enable_router_replay and self.model.impl not in ("custom", "auto"):
            raise ValueError("router replay is only supported with the custom implementation or auto mode")
        return self
