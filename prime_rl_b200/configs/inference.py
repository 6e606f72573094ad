"""Inference (rollout engine) configuration. Field names follow the reference's
``configs/inference.py``; the ``vllm`` block keeps its name for TOML compatibility and
configures this repository's own engine (``prime_rl_b200/engine``)."""

from __future__ import annotations

from pathlib import Path
from typing import Annotated, Any, Literal, TypeAlias

from pydantic import Field, model_validator

from .base import BaseConfig
from .shared import VLMConfig, EnvVars, LogConfig, SlurmConfig, default_output_dir


class ServerConfig(BaseConfig):
    host: str | None = None
    port: int = 8000
    liveness_timeout_seconds: float = Field(30.0, gt=0)


class EngineConfig(BaseConfig):
    """Engine arguments under the names the reference's ``[inference.vllm]`` block uses
    (packages/prime-rl-configs/src/prime_rl/configs/inference.py:42-210). The typed fields are the ones
    this engine reads; any other key is accepted and kept (``extra``), as the reference passes unknown keys
    through to its serving engine: kebab-case keys become snake_case and string values from the command
    line are JSON-parsed where they parse."""

    model_config = {**BaseConfig.model_config, "extra": "allow"}

    @model_validator(mode="before")
    @classmethod
    def _normalise_extras(cls, data):
        if not isinstance(data, dict):
            return data
        import json

        out = {}
        for key, value in data.items():
            if key in cls.model_fields:
                out[key] = value
                continue
            if isinstance(value, str):
                try:
                    value = json.loads(value)
                except ValueError:
                    pass
            out[key.replace("-", "_")] = value
        return out

    model: str = "Qwen/Qwen3-0.6B"
    dtype: Literal["auto", "float16", "bfloat16", "float32"] = "auto"
    max_model_len: int | None = None
    enforce_eager: bool = False
    trust_remote_code: bool = False
    chat_template: str | None = None
    tool_call_parser: str | None = "auto"
    reasoning_parser: str | None = "auto"
    rope_scaling: dict[str, Any] | str | None = None
    tensor_parallel_size: int = 1
    data_parallel_size: int = Field(1, ge=1)
    data_parallel_size_local: int | None = Field(None, ge=1)
    data_parallel_rpc_port: int = Field(13345, ge=1, le=65535)
    api_server_count: int = Field(1, ge=0)
    seed: int = 0
    gpu_memory_utilization: float = 0.9
    enable_prefix_caching: bool | None = None
    quantization: str | None = None            # None | "fp8" (128x128 weight blocks, 1x128 activation scales)
    enable_lora: bool = False
    max_loras: int = 1
    max_lora_rank: int | None = None
    lora_target_modules: list[str] | None = None
    # vision tower for image inputs (same description as ``model.vlm`` of the trainer); None: text only
    vlm: VLMConfig | None = None
    enable_expert_parallel: bool = False
    all2all_backend: str = "allgather_reducescatter"
    enable_eplb: bool = False
    enable_dbo: bool = False
    enable_return_routed_experts: bool = False
    # engine-specific
    page_size: int = 16
    num_pages: int | None = None               # None: sized from gpu_memory_utilization
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 16384
    arch: dict[str, Any] | None = None         # inline architecture for random-init runs
    random_init: bool = False


class WeightBroadcastConfig(BaseConfig):
    type: Literal["nccl", "filesystem", "nixl", "p2p"] = "filesystem"


class CPUOffloadTier(BaseConfig):
    num_bytes: int = Field(..., gt=0)


class DiskOffloadTier(BaseConfig):
    path: Path


class NativeKVCacheOffloadConfig(BaseConfig):
    type: Literal["native"] = "native"
    cpu: CPUOffloadTier | None = None
    disk: DiskOffloadTier | None = None


class MooncakeKVCacheOffloadConfig(BaseConfig):
    type: Literal["mooncake"] = "mooncake"
    cpu: CPUOffloadTier | None = None
    disk: DiskOffloadTier | None = None
    device_name: str = ""


KVCacheOffloadConfig: TypeAlias = Annotated[NativeKVCacheOffloadConfig | MooncakeKVCacheOffloadConfig,
                                            Field(discriminator="type")]


class VllmRouterConfig(BaseConfig):
    """Consistent-hash request router in front of several engine replicas."""

    type: Literal["vllm-router"] = "vllm-router"
    policy: str = "consistent_hash"


class LlmdRouterConfig(BaseConfig):
    type: Literal["llm-d"] = "llm-d"
    scorers: dict[str, float] = {"prefix-cache-scorer": 2.0, "queue-scorer": 1.0}
    prefill_scorer_overrides: dict[str, float] = {}
    decode_scorer_overrides: dict[str, float] = {}
    non_cached_tokens: int = 16
    decode_sidecar_port: int = 8300


RouterConfig: TypeAlias = Annotated[VllmRouterConfig | LlmdRouterConfig, Field(discriminator="type")]


class SingleNodeInferenceDeploymentConfig(BaseConfig):
    type: Literal["single_node"] = "single_node"
    gpus_per_node: int = 8


class MultiNodeInferenceDeploymentConfig(BaseConfig):
    type: Literal["multi_node"] = "multi_node"
    gpus_per_node: int = 8
    num_nodes: int = Field(2, ge=1)


class DisaggregatedInferenceDeploymentConfig(BaseConfig):
    type: Literal["disaggregated"] = "disaggregated"
    gpus_per_node: int = 8
    prefill_nodes_per_replica: int = Field(1, ge=1)
    decode_nodes_per_replica: int = Field(1, ge=1)
    num_prefill_replicas: int = Field(1, ge=1)
    num_decode_replicas: int = Field(1, ge=1)
    prefill_port: int = 8100
    decode_port: int = 8200
    prefill_env_vars: EnvVars = {}
    decode_env_vars: EnvVars = {}
    prefill_vllm_overrides: dict[str, Any] = {}
    decode_vllm_overrides: dict[str, Any] = {}


InferenceDeploymentConfig: TypeAlias = Annotated[
    SingleNodeInferenceDeploymentConfig | MultiNodeInferenceDeploymentConfig
    | DisaggregatedInferenceDeploymentConfig, Field(discriminator="type")]


class InferenceConfig(BaseConfig):
    server: ServerConfig = ServerConfig()
    router: RouterConfig | None = None
    backend_port: int = 8100
    vllm: EngineConfig = Field(default_factory=EngineConfig)
    log: LogConfig = LogConfig()
    env_vars: EnvVars = {}
    use_deep_gemm: bool = False
    weight_broadcast: WeightBroadcastConfig = WeightBroadcastConfig()
    kv_cache_offload: KVCacheOffloadConfig | None = None
    use_pd_kv_transfer: bool = False
    enable_return_sampling_mask: bool = False
    enable_fp32_lm_head: bool = True              # the LM head of this engine always accumulates in fp32
    enable_fp32_router_logits: bool = True        # router logits are fp32 here as well
    deployment: InferenceDeploymentConfig = SingleNodeInferenceDeploymentConfig()
    slurm: SlurmConfig | None = None
    output_dir: Path = Field(default_factory=default_output_dir)
    dry_run: bool = False
