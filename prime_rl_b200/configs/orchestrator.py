"""Orchestrator configuration (field names follow the reference's ``configs/orchestrator.py``).

Environments: the reference loads ``verifiers`` environments served by env-server
processes; that package is not available offline, so an environment here is named by
``id`` from the built-in registry (``prime_rl_b200/orchestrator/envs.py``) or by an
``import_path`` to a factory, with free-form ``args``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Annotated, Any, Literal, TypeAlias

from pydantic import Field, model_validator

from .algorithm import AlgoConfig, GRPOAlgoConfig
from .base import BaseConfig
from .monitors import MonitorsConfig
from .shared import (BaseModelConfig, BaseWeightBroadcastConfig, ClientConfig, EnvVars, HeartbeatConfig, LogConfig,
                     ResumeConfig, TransportConfig, ZMQTransportConfig, default_output_dir)
from .trainer import TokenizerConfig

TRAIN_TOP_K_BOUND = 512


class LoRAConfig(BaseConfig):
    rank: int | None = Field(None, ge=1)
    alpha: float | None = Field(None, ge=0)


class ModelConfig(BaseModelConfig):
    lora: LoRAConfig | None = None
    client: ClientConfig = ClientConfig()


class TrainSamplingConfig(BaseConfig):
    temperature: float = Field(1.0, ge=0, le=2.0)
    top_p: float = Field(1.0, gt=0, le=1.0)
    top_k: int | None = Field(None, ge=1)
    max_completion_tokens: int | None = None
    extra_body: dict[str, Any] = {}

    @model_validator(mode="after")
    def _bound_top_k(self):
        if self.top_k is not None and self.top_k > TRAIN_TOP_K_BOUND:
            raise ValueError(f"top_k must not exceed {TRAIN_TOP_K_BOUND} (bounds the sampling-mask size)")
        if self.top_p < 1.0 and self.top_k is None:
            self.top_k = TRAIN_TOP_K_BOUND
        return self

    @property
    def truncated(self) -> bool:
        return self.top_p < 1.0 or self.top_k is not None


class EvalSamplingConfig(BaseConfig):
    temperature: float | None = Field(None, ge=0, le=2.0)
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = Field(None, ge=0)
    max_completion_tokens: int | None = None
    reasoning_effort: Literal["minimal", "low", "medium", "high"] | None = None
    extra_body: dict[str, Any] = {}


class EnvServeConfig(BaseConfig):
    """Where the environment of a source is served. ``address`` set: an externally managed env server;
    unset: the launcher spawns one at ``tcp://127.0.0.1:<env_server_base_port + index>``."""

    model_config = {**BaseConfig.model_config, "extra": "allow"}
    address: str | None = None
    num_workers: int | None = None


class RendererConfig(BaseConfig):
    """Chat renderer selection. ``name = "auto"`` picks by model name; other names and their options are
    passed through to the renderer registry untouched (the reference takes this block from the external
    ``renderers`` package: packages/prime-rl-configs/src/prime_rl/configs/orchestrator.py:507)."""

    model_config = {**BaseConfig.model_config, "extra": "allow"}
    name: str = "auto"


class EnvConfig(BaseConfig):
    """One environment. Two spellings are accepted:

    * this framework's own: ``id`` from the built-in registry (``orchestrator/envs.py``) or an
      ``import_path`` to a factory, with free-form ``args``;
    * the reference's ``env.*`` tree (``env.taskset.id``, ``env.agent.harness.id``, ...), which belongs to the
      external ``verifiers`` package there and is kept as an opaque mapping here; ``env.taskset.id`` (or
      ``env.id``) names the environment and ``env.taskset.args`` / ``env.args`` feed its factory."""

    id: str = "reverse-text"
    import_path: str | None = None
    args: dict[str, Any] = {}
    env: dict[str, Any] = {}
    serve: EnvServeConfig = EnvServeConfig()
    name: str | None = None
    ratio: float = Field(1.0, gt=0)

    @model_validator(mode="after")
    def _from_env_tree(self):
        tree = self.env or {}
        taskset = tree.get("taskset") if isinstance(tree.get("taskset"), dict) else {}
        ident = taskset.get("id") or tree.get("id")
        if ident and "id" not in self.model_fields_set:
            self.id = str(ident)
        extra = taskset.get("args") or tree.get("args")
        if isinstance(extra, dict) and "args" not in self.model_fields_set:
            self.args = dict(extra)
        return self

    @property
    def resolved_name(self) -> str:
        return self.name or self.id


class StandardSamplerConfig(BaseConfig):
    type: Literal["standard"] = "standard"


class DifficultyPoolConfig(BaseConfig):
    threshold: float
    weight: float = Field(ge=0)


def default_difficulty_pools() -> dict[str, DifficultyPoolConfig]:
    return {"easy": DifficultyPoolConfig(threshold=0.8, weight=0.2),
            "normal": DifficultyPoolConfig(threshold=0.2, weight=0.6),
            "hard": DifficultyPoolConfig(threshold=0.0, weight=0.2)}


class DifficultyPoolSamplerConfig(BaseConfig):
    type: Literal["difficulty_pool"] = "difficulty_pool"
    pools: dict[str, DifficultyPoolConfig] = Field(default_factory=default_difficulty_pools)
    seed: int = 42


TaskSamplerConfig: TypeAlias = Annotated[StandardSamplerConfig | DifficultyPoolSamplerConfig,
                                         Field(discriminator="type")]


class AdvRangeGateConfig(BaseConfig):
    """Rejects groups whose advantages all fall inside [reject_min, reject_max] (e.g. all zero)."""

    type: Literal["advantage_range"] = "advantage_range"
    reject_min: float = 0.0
    reject_max: float = 0.0


AdmissionGateConfig: TypeAlias = Annotated[AdvRangeGateConfig, Field(discriminator="type")]


class CurriculumConfig(BaseConfig):
    sampler: TaskSamplerConfig = Field(default_factory=StandardSamplerConfig)
    gates: dict[str, AdmissionGateConfig] = Field(default_factory=dict)


class TrainSourceConfig(EnvConfig):
    sampling: TrainSamplingConfig | None = None
    group_size: int | None = Field(None, ge=1)
    algo: AlgoConfig | None = None
    curriculum: CurriculumConfig | None = None


class EvalSourceConfig(EnvConfig):
    sampling: EvalSamplingConfig = EvalSamplingConfig()
    num_examples: int = -1
    group_size: int = Field(1, ge=1)
    interval: int = Field(100, ge=1)


class TrainConfig(BaseConfig):
    source: list[TrainSourceConfig] = Field(default_factory=lambda: [TrainSourceConfig()])
    sampling: TrainSamplingConfig = TrainSamplingConfig()


class EvalConfig(BaseConfig):
    source: list[EvalSourceConfig] = Field(default_factory=list)
    sampling: EvalSamplingConfig = Field(default_factory=EvalSamplingConfig)
    num_examples: int = -1
    group_size: int = Field(1, ge=1)
    interval: int = Field(100, ge=1)
    skip_first_step: bool = False
    retrigger_on_resume: bool = False


class CheckpointConfig(BaseConfig):
    interval: int | None = Field(None, ge=1)
    wait_for_weights_timeout: int | None = Field(None, ge=1)
    keep_last: int | None = Field(None, ge=1)
    keep_interval: int | None = Field(None, ge=1)
    skip_progress: bool = False


class FileSystemWeightBroadcastConfig(BaseWeightBroadcastConfig):
    type: Literal["filesystem"] = "filesystem"


class InMemoryWeightBroadcastConfig(BaseWeightBroadcastConfig):
    host: str = "localhost"
    port: int
    inference_world_size: int = Field(1, ge=1)


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
    type: Literal["p2p"] = "p2p"
    port: int = 29502
    quantize_in_weight_transfer: bool = False

    @property
    def quantize(self) -> str | None:
        """"fp8": 2-D weights are quantised to block-scaled fp8 in flight."""
        return "fp8" if self.quantize_in_weight_transfer else None


WeightBroadcastConfig: TypeAlias = Annotated[
    FileSystemWeightBroadcastConfig | NCCLWeightBroadcastConfig | NIXLWeightBroadcastConfig
    | P2PWeightBroadcastConfig, Field(discriminator="type")]


class ConcurrencyConfig(BaseConfig):
    initial_inflight: int | None = Field(None, ge=1)
    min_inflight: int = Field(1, ge=1)
    max_inflight: int | None = Field(1024, ge=1)

    @model_validator(mode="after")
    def _bounds(self):
        if self.max_inflight is not None:
            if self.initial_inflight is not None and self.initial_inflight > self.max_inflight:
                raise ValueError("concurrency.initial_inflight must not exceed concurrency.max_inflight")
            if self.min_inflight > self.max_inflight:
                raise ValueError("concurrency.min_inflight must not exceed concurrency.max_inflight")
        return self


class OrchestratorConfig(BaseConfig):
    algo: AlgoConfig = GRPOAlgoConfig()
    model: ModelConfig = ModelConfig()
    train: TrainConfig = TrainConfig()
    tokenizer: TokenizerConfig = TokenizerConfig()
    renderer: RendererConfig = RendererConfig()
    eval: EvalConfig | None = None
    log: LogConfig = LogConfig()
    env_vars: EnvVars = {}
    monitors: MonitorsConfig = MonitorsConfig()
    collect_inference_metrics: bool = True
    inference_metrics_roles: list[Literal["prefill", "decode"]] | None = None
    ckpt: CheckpointConfig | None = None
    resume: ResumeConfig | None = None
    weight_broadcast: WeightBroadcastConfig = FileSystemWeightBroadcastConfig()
    rollout_transport: TransportConfig = ZMQTransportConfig()
    output_dir: Path = Field(default_factory=default_output_dir)
    tasks_per_minute: int | None = Field(None, ge=1)
    env_server_base_port: int = Field(5000, ge=1, le=65535)
    batch_size: int | None = Field(None, ge=1)
    constant_trainer_batch_size: bool = True
    token_batch_size: int | None = Field(None, ge=1)
    concurrency: ConcurrencyConfig = ConcurrencyConfig()
    group_size: int = Field(1, ge=1)
    seq_len: int = 2048
    num_train_workers: int = Field(1, ge=1)
    pad_to_multiple_of: int = Field(1, ge=1)
    max_steps: int | None = None
    max_off_policy_steps: int = Field(8, ge=0)
    heartbeat: HeartbeatConfig | None = None
    enable_return_routed_experts: bool = False
    # The built-in token-level environments run inside the orchestrator process. With this switch (or a
    # source's ``serve.spawn = true``) the ``rl`` launcher starts one env-server process per train / eval source
    # at ``http://127.0.0.1:<env_server_base_port + index>`` and the orchestrator talks to it over HTTP, which
    # is how heavy or sandboxed environments are kept off the orchestrator's event loop.
    spawn_env_servers: bool = False
    seed: int = 0
    dry_run: bool = False

    @model_validator(mode="after")
    def _checks(self):
        if self.batch_size is None and self.token_batch_size is None:
            self.batch_size = 32
        if self.batch_size is not None and self.token_batch_size is not None:
            raise ValueError("set either batch_size (traces per step) or token_batch_size, not both")
        if self.batch_size is not None and self.batch_size % self.group_size:
            raise ValueError("batch_size must be a multiple of group_size")
        if self.tokenizer.name is None:
            self.tokenizer.name = self.model.name
        if self.train.sampling.truncated and self.train.sampling.top_k and self.train.sampling.top_k > TRAIN_TOP_K_BOUND:
            raise ValueError(f"top_k must be <= {TRAIN_TOP_K_BOUND}")
        return self

    @property
    def env_addresses(self) -> dict[tuple[str, str], str]:
        """(kind, source name) -> address of the source's env server: its explicit ``serve.address`` (an
        externally managed server) or the port derived from ``env_server_base_port`` and the source's index,
        train sources first (reference: configs/orchestrator.py ``env_addresses``)."""
        out: dict[tuple[str, str], str] = {}
        sources = [("train", s) for s in self.train.source] + [("eval", s) for s in (self.eval.source if self.eval else [])]
        for index, (kind, s) in enumerate(sources):
            out[(kind, s.resolved_name)] = s.serve.address or f"http://127.0.0.1:{self.env_server_base_port + index}"
        return out

    def spawned_sources(self) -> list[tuple[str, object, str]]:
        """(kind, source, address) of every source the launcher has to start an env server for."""
        addrs = self.env_addresses
        sources = [("train", s) for s in self.train.source] + [("eval", s) for s in (self.eval.source if self.eval else [])]
        return [(kind, s, addrs[(kind, s.resolved_name)]) for kind, s in sources
                if s.serve.address is None and (self.spawn_env_servers or getattr(s.serve, "spawn", False))
                and s.id != "remote"]

    def source_group_size(self, src: TrainSourceConfig) -> int:
        return src.group_size or self.group_size

    def source_algo(self, src: TrainSourceConfig):
        return src.algo or self.algo

    def source_sampling(self, src: TrainSourceConfig) -> TrainSamplingConfig:
        return src.sampling or self.train.sampling
