"""``rl`` launcher configuration: a shared top level that is copied into the trainer /
orchestrator / inference sub-configs, then cross-wired (reference:
packages/prime-rl-configs/src/prime_rl/configs/rl.py:235-897, utils/validation.py)."""

from __future__ import annotations

import uuid
from pathlib import Path
from typing import Annotated, Any, Literal, TypeAlias

from pydantic import Field, model_validator

from .base import BaseConfig, deep_merge
from .inference import InferenceConfig
from .monitors import FileMonitorConfig, PrimeMonitorConfig
from .orchestrator import OrchestratorConfig
from .shared import EnvVars, ResumeConfig, RunConfig, SlurmConfig, TransportConfig, VLMConfig, default_output_dir
from .trainer import TokenizerConfig, TrainerConfig


class SharedLogConfig(BaseConfig):
    level: str | None = None
    json_logging: bool = False


class SharedWandbConfig(BaseConfig):
    project: str | None = "prime-rl"
    entity: str | None = None
    name: str | None = None
    group: str | None = None
    tags: list[str] | None = None
    offline: bool | None = False


class SharedMonitorsConfig(BaseConfig):
    wandb: SharedWandbConfig | None = None
    file: FileMonitorConfig | None = None
    prime: PrimeMonitorConfig | None = None


class SharedCheckpointConfig(BaseConfig):
    output_dir: Path | None = None
    interval: int | None = None
    keep_last: int | None = Field(None, ge=1)
    keep_interval: int | None = Field(None, ge=1)


class SharedModelConfig(BaseConfig):
    name: str = "Qwen/Qwen3-0.6B"
    vlm: VLMConfig | None = None
    arch: dict[str, Any] | None = None


class SharedFileSystemWeightBroadcastConfig(BaseConfig):
    type: Literal["filesystem"] = "filesystem"
    timeout: int = 1200


class SharedNCCLWeightBroadcastConfig(BaseConfig):
    type: Literal["nccl"] = "nccl"
    host: str = "localhost"
    port: int = 29501
    timeout: int = 1200
    quantize_in_weight_transfer: bool = False


class SharedNIXLWeightBroadcastConfig(BaseConfig):
    type: Literal["nixl"] = "nixl"
    host: str = "localhost"
    port: int = 8001
    timeout: int = 1200
    session_id: str = "default"
    overlap_transfer_and_replay: bool = False


class SharedP2PWeightBroadcastConfig(BaseConfig):
    type: Literal["p2p"] = "p2p"
    host: str = "localhost"
    port: int = 29502
    timeout: int = 1200
    quantize_in_weight_transfer: bool = True


SharedWeightBroadcastConfig: TypeAlias = Annotated[
    SharedFileSystemWeightBroadcastConfig | SharedNCCLWeightBroadcastConfig | SharedNIXLWeightBroadcastConfig
    | SharedP2PWeightBroadcastConfig, Field(discriminator="type")]


class SingleNodeDeploymentConfig(BaseConfig):
    type: Literal["single_node"] = "single_node"
    gpus_per_node: int = 8
    num_train_gpus: int = 1
    num_infer_gpus: int = 1


class MultiNodeDeploymentConfig(BaseConfig):
    type: Literal["multi_node"] = "multi_node"
    gpus_per_node: int = 8
    num_train_nodes: int
    num_infer_nodes: int | None = Field(None, ge=0)
    num_infer_replicas: int = Field(1, ge=1)
    nodes_per_fsdp_group: int | None = None
    orchestrator_on_inference: bool = False


DeploymentConfig: TypeAlias = Annotated[SingleNodeDeploymentConfig | MultiNodeDeploymentConfig,
                                        Field(discriminator="type")]

_SHARED_TO_SUB = ("max_steps", "resume")


class RLConfig(BaseConfig):
    trainer: TrainerConfig = Field(default_factory=TrainerConfig)
    orchestrator: OrchestratorConfig = Field(default_factory=OrchestratorConfig)
    inference: InferenceConfig | None = None
    env_vars: EnvVars = {}
    run: RunConfig = Field(default_factory=RunConfig)
    output_dir: Path = Field(default_factory=default_output_dir)
    clean: bool = False
    log: SharedLogConfig = SharedLogConfig()
    ckpt: SharedCheckpointConfig | None = None
    resume: ResumeConfig | None = None
    monitors: SharedMonitorsConfig = SharedMonitorsConfig()
    model: SharedModelConfig | None = None
    tokenizer: TokenizerConfig | None = None
    max_steps: int | None = None
    seq_len: int | None = None
    weight_broadcast: SharedWeightBroadcastConfig | None = None
    rollout_transport: TransportConfig | None = None
    deployment: DeploymentConfig = SingleNodeDeploymentConfig()
    slurm: SlurmConfig | None = None
    dashboard: bool = True
    dry_run: bool = False

    # ------------------------------------------------------------------ shared -> sub-configs
    @model_validator(mode="before")
    @classmethod
    def _propagate_shared(cls, data):
        if not isinstance(data, dict):
            return data
        data = dict(data)
        subs = {k: dict(data.get(k) or {}) for k in ("trainer", "orchestrator")}
        inf = data.get("inference")
        inf = dict(inf) if isinstance(inf, dict) else inf

        def push(sub: dict, path: list[str], value):
            cur = sub
            for p in path[:-1]:
                cur = cur.setdefault(p, {}) if isinstance(cur.get(p), dict) or p not in cur else cur[p]
            cur.setdefault(path[-1], value)

        if data.get("model"):
            m = data["model"]
            for sub in subs.values():
                sub["model"] = deep_merge({k: v for k, v in m.items() if v is not None}, sub.get("model") or {})
            subs["orchestrator"]["model"].pop("arch", None)
            if isinstance(inf, dict):
                v = dict(inf.get("vllm") or {})
                v.setdefault("model", m.get("name"))
                if m.get("arch"):
                    v.setdefault("arch", m["arch"])
                inf["vllm"] = v
        for key in ("max_steps", "resume", "rollout_transport", "weight_broadcast", "tokenizer"):
            if data.get(key) is not None:
                for name, sub in subs.items():
                    val = data[key]
                    if key == "weight_broadcast" and isinstance(val, dict):
                        val = dict(val)
                    sub.setdefault(key, val)
        if data.get("weight_broadcast") and isinstance(inf, dict):
            inf.setdefault("weight_broadcast", {"type": data["weight_broadcast"].get("type", "filesystem")})
        if data.get("seq_len") is not None:
            subs["trainer"].setdefault("model", {}).setdefault("seq_len", data["seq_len"])
            subs["orchestrator"].setdefault("seq_len", data["seq_len"])
        if data.get("ckpt"):
            ck = {k: v for k, v in data["ckpt"].items() if v is not None}
            subs["trainer"]["ckpt"] = deep_merge(ck, subs["trainer"].get("ckpt") or {})
            o = {k: v for k, v in ck.items() if k in ("interval", "keep_last", "keep_interval")}
            subs["orchestrator"]["ckpt"] = deep_merge(o, subs["orchestrator"].get("ckpt") or {})
        if data.get("log"):
            for sub in list(subs.values()) + ([inf] if isinstance(inf, dict) else []):
                lg = dict(sub.get("log") or {})
                if data["log"].get("level") is not None:
                    lg.setdefault("level", data["log"]["level"])
                lg.setdefault("json_logging", data["log"].get("json_logging", False))
                sub["log"] = lg
        if data.get("monitors"):
            mon = {k: v for k, v in data["monitors"].items() if v is not None and k != "wandb"}
            if data["monitors"].get("wandb"):
                w = data["monitors"]["wandb"]
                mon["wandb"] = {k: w[k] for k in ("project", "entity", "name", "offline") if w.get(k) is not None}
            for sub in subs.values():
                sub["monitors"] = deep_merge(mon, sub.get("monitors") or {})
        data["trainer"], data["orchestrator"] = subs["trainer"], subs["orchestrator"]
        if inf is not None:
            data["inference"] = inf
        return data

    # ------------------------------------------------------------------ cross-wiring
    @model_validator(mode="after")
    def _wire(self):
        t, o, i, d = self.trainer, self.orchestrator, self.inference, self.deployment
        if self.run.name is None:
            env = "-".join(s.resolved_name for s in o.train.source) or "env"
            self.run.name = f"{env}--{Path(t.model.name).name}--{uuid.uuid4().hex[:6]}"
        run_dir = self.output_dir / (self.run.dir or self.run.name)
        t.output_dir = o.output_dir = run_dir
        if i is not None:
            i.output_dir = run_dir
        # LoRA adapters are loaded from disk by the engine
        if t.model.lora is not None and t.weight_broadcast.type != "filesystem":
            raise ValueError("LoRA requires weight_broadcast.type = 'filesystem'")
        if t.weight_broadcast.type != o.weight_broadcast.type:
            raise ValueError("trainer and orchestrator must use the same weight_broadcast.type")
        if t.rollout_transport.type != o.rollout_transport.type:
            raise ValueError("trainer and orchestrator must use the same rollout_transport.type")
        if o.model.name != t.model.name:
            raise ValueError("trainer and orchestrator must train / sample the same model")
        if o.seq_len != t.model.seq_len:
            o.seq_len = t.model.seq_len
        if isinstance(d, SingleNodeDeploymentConfig):
            cp = t.model.cp
            if d.num_train_gpus % cp:
                raise ValueError("num_train_gpus must be a multiple of trainer.model.cp")
            o.num_train_workers = max(1, d.num_train_gpus // cp)
            o.pad_to_multiple_of = max(o.pad_to_multiple_of, cp)
            if i is not None:
                tp = i.vllm.tensor_parallel_size
                if d.num_infer_gpus % tp:
                    raise ValueError("num_infer_gpus must be a multiple of inference tensor_parallel_size")
                i.vllm.data_parallel_size = max(1, d.num_infer_gpus // tp)
                if tp > 1 and getattr(t.weight_broadcast, "type", "filesystem") != "filesystem":
                    # only rank 0 of a tensor-parallel engine answers the admin routes; every rank loads its
                    # slices from the checkpoint directory
                    raise ValueError("tensor-parallel inference engines take weight updates through "
                                     "weight_broadcast.type = 'filesystem'")
                if hasattr(t.weight_broadcast, "inference_world_size"):
                    t.weight_broadcast.inference_world_size = d.num_infer_gpus
                    if hasattr(o.weight_broadcast, "inference_world_size"):
                        o.weight_broadcast.inference_world_size = d.num_infer_gpus
        if t.enable_router_replay:
            o.enable_return_routed_experts = True
            if i is not None:
                i.vllm.enable_return_routed_experts = True
        if o.train.sampling.truncated and i is not None:
            i.enable_return_sampling_mask = True
        if i is not None:
            base = f"http://localhost:{i.server.port}/v1"
            if o.model.client.base_url == "http://localhost:8000/v1":
                o.model.client.base_url = base
            if o.model.client.admin_base_url is None:
                o.model.client.admin_base_url = [base]
            if i.vllm.model != t.model.name:
                i.vllm.model = t.model.name
        if o.max_steps is None and t.max_steps is not None:
            o.max_steps = t.max_steps
        return self

    @property
    def run_dir(self) -> Path:
        return self.output_dir / (self.run.dir or self.run.name)
