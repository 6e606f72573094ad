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

        if isinstance(data.get("model"), dict) and data["model"]:
            m = data["model"]
            for sub in subs.values():
                sub["model"] = deep_merge({k: v for k, v in m.items() if v is not None}, sub.get("model") or {})
            subs["orchestrator"]["model"].pop("arch", None)
            if isinstance(inf, dict):
                v = dict(inf.get("vllm") or {})
                v.setdefault("model", m.get("name"))
                if m.get("arch"):
                    v.setdefault("arch", m["arch"])
                if m.get("vlm"):
                    v.setdefault("vlm", m["vlm"])           # the engine runs the same vision tower on image inputs
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
    # What the launcher derives once all three sub-configs exist (behaviour of the reference's validators:
    # packages/prime-rl-configs/src/prime_rl/configs/rl.py:399-445 run identity, :459-516 weight broadcast,
    # :519-540 rollout transport, :556-600 LoRA, :602-673 router replay / sampling mask, :718-826 deployment,
    # :861-885 inference client).
    @model_validator(mode="after")
    def _wire(self):
        self._wire_run_identity()
        self._wire_lora()
        self._wire_weight_broadcast()
        self._wire_rollout_transport()
        self._wire_deployment()
        self._wire_replay_and_masks()
        self._wire_inference_client()
        t, o = self.trainer, self.orchestrator
        if o.seq_len != t.model.seq_len:
            o.seq_len = t.model.seq_len
        if o.max_steps is None and t.max_steps is not None:
            o.max_steps = t.max_steps
        return self

    def _wire_run_identity(self) -> None:
        t, o, i = self.trainer, self.orchestrator, self.inference
        if self.run.name is None:
            env = "-".join(s.resolved_name for s in o.train.source) or "env"
            self.run.name = f"{env}--{Path(t.model.name).name}--{uuid.uuid4().hex[:6]}"
        run_dir = self.output_dir / (self.run.dir or self.run.name)
        t.output_dir = o.output_dir = run_dir
        if i is not None:
            i.output_dir = run_dir
        for mon in (self.monitors, t.monitors, o.monitors):          # unnamed W&B / platform runs take the run name
            for sink in (getattr(mon, "wandb", None), getattr(mon, "prime", None)):
                if sink is not None and getattr(sink, "name", "unset") is None:
                    sink.name = self.run.name

    def _wire_lora(self) -> None:
        t, o, i = self.trainer, self.orchestrator, self.inference
        lora = t.model.lora
        if lora is None:
            return
        from .orchestrator import LoRAConfig as OrchestratorLoRAConfig

        if o.model.lora is None:
            o.model.lora = OrchestratorLoRAConfig()
        for key in ("rank", "alpha"):
            mine, theirs = getattr(o.model.lora, key), getattr(lora, key)
            if mine is not None and mine != theirs:
                raise ValueError(f"orchestrator.model.lora.{key} ({mine}) conflicts with trainer.model.lora.{key} "
                                 f"({theirs}): remove it to inherit the trainer's value")
            setattr(o.model.lora, key, theirs)
        if i is not None:
            i.vllm.enable_lora = True
            i.vllm.max_lora_rank = lora.rank

    def _wire_weight_broadcast(self) -> None:
        """No ``weight_broadcast`` given: in-memory (NCCL) when the launcher also runs an inference server,
        files when adapters are trained (engines load adapters from a directory) or when there is no
        inference block."""
        t, o, i = self.trainer, self.orchestrator, self.inference
        if self.weight_broadcast is None:
            explicit = "weight_broadcast" in t.model_fields_set or "weight_broadcast" in o.model_fields_set
            if explicit:
                kind = t.weight_broadcast.type
            elif t.model.lora is not None or i is None:
                kind = "filesystem"
            else:
                kind = "nccl"
            shared = {"filesystem": SharedFileSystemWeightBroadcastConfig, "nccl": SharedNCCLWeightBroadcastConfig,
                      "nixl": SharedNIXLWeightBroadcastConfig, "p2p": SharedP2PWeightBroadcastConfig}[kind]
            if explicit:
                self.weight_broadcast = shared(**{k: v for k, v in t.weight_broadcast.model_dump().items()
                                                  if k in shared.model_fields})
            else:
                self.weight_broadcast = shared()
        wb = self.weight_broadcast
        if wb.type != "filesystem" and t.model.lora is not None:
            raise ValueError("LoRA requires weight_broadcast.type = 'filesystem': engines load adapters from a "
                             "PEFT-shaped directory on disk")
        from . import orchestrator as oc
        from . import trainer as tc

        if wb.type == "filesystem":
            t.weight_broadcast = tc.FileSystemWeightBroadcastConfig(timeout=wb.timeout)
            o.weight_broadcast = oc.FileSystemWeightBroadcastConfig(timeout=wb.timeout)
        else:
            world = (i.vllm.data_parallel_size * i.vllm.tensor_parallel_size) if i is not None else 1
            common = dict(host=wb.host, port=wb.port, timeout=wb.timeout, inference_world_size=world)
            extra = {k: getattr(wb, k) for k in ("quantize_in_weight_transfer", "session_id",
                                                 "overlap_transfer_and_replay") if hasattr(wb, k)}
            names = {"nccl": "NCCLWeightBroadcastConfig", "nixl": "NIXLWeightBroadcastConfig",
                     "p2p": "P2PWeightBroadcastConfig"}[wb.type]
            t.weight_broadcast = getattr(tc, names)(**common, **extra)
            o.weight_broadcast = getattr(oc, names)(**common, **extra)
        if i is not None:
            i.weight_broadcast.type = wb.type

    def _wire_rollout_transport(self) -> None:
        t, o = self.trainer, self.orchestrator
        if self.rollout_transport is None:
            # one side set explicitly wins; otherwise both keep their (equal) defaults
            if "rollout_transport" in t.model_fields_set and "rollout_transport" not in o.model_fields_set:
                o.rollout_transport = t.rollout_transport.model_copy()
            elif "rollout_transport" in o.model_fields_set and "rollout_transport" not in t.model_fields_set:
                t.rollout_transport = o.rollout_transport.model_copy()
            self.rollout_transport = t.rollout_transport
        if t.rollout_transport.type != o.rollout_transport.type:
            raise ValueError("trainer and orchestrator must use the same rollout_transport.type")

    def _wire_deployment(self) -> None:
        t, o, i, d = self.trainer, self.orchestrator, self.inference, self.deployment
        cp = t.model.cp
        o.pad_to_multiple_of = max(o.pad_to_multiple_of, cp)
        if isinstance(d, SingleNodeDeploymentConfig):
            if d.num_train_gpus % cp:
                raise ValueError("num_train_gpus must be a multiple of trainer.model.cp")
            if d.num_train_gpus > 1:
                o.num_train_workers = d.num_train_gpus // cp       # one batch writer slot per data replica
            if i is not None:
                tp = i.vllm.tensor_parallel_size
                if d.num_infer_gpus != i.vllm.data_parallel_size * tp:
                    if d.num_infer_gpus % tp:
                        raise ValueError("num_infer_gpus must be a multiple of inference tensor_parallel_size")
                    i.vllm.data_parallel_size = d.num_infer_gpus // tp
                if i.vllm.api_server_count < i.vllm.data_parallel_size and not i.vllm.enable_lora:
                    i.vllm.api_server_count = i.vllm.data_parallel_size
                world = i.vllm.data_parallel_size * tp
        else:
            o.num_train_workers = d.num_train_nodes * d.gpus_per_node // cp
            if d.nodes_per_fsdp_group is not None:
                if d.num_train_nodes % d.nodes_per_fsdp_group:
                    raise ValueError(f"deployment.num_train_nodes ({d.num_train_nodes}) must be divisible by "
                                     f"deployment.nodes_per_fsdp_group ({d.nodes_per_fsdp_group})")
                t.model.dp_replicate = d.num_train_nodes // d.nodes_per_fsdp_group
            world = None
            if i is not None and i.deployment.type != "disaggregated":
                tp = i.vllm.tensor_parallel_size
                if d.gpus_per_node % tp:
                    raise ValueError("deployment.gpus_per_node must be divisible by inference tensor_parallel_size")
                per_node = d.gpus_per_node // tp
                if i.vllm.data_parallel_size == 1 and per_node > 1:
                    i.vllm.data_parallel_size = per_node
                if i.vllm.data_parallel_size_local is None and per_node > 1:
                    i.vllm.data_parallel_size_local = per_node
                if i.vllm.api_server_count == 1 and per_node > 1:
                    i.vllm.api_server_count = per_node
            infer_nodes = (d.num_infer_nodes or 0) * max(1, d.num_infer_replicas) if d.num_infer_nodes else 0
            if infer_nodes:
                world = infer_nodes * d.gpus_per_node            # every allocated inference GPU is a transfer worker
                if getattr(t.weight_broadcast, "type", "") == "nccl":
                    t.weight_broadcast.host = "0.0.0.0"
        if i is not None or not isinstance(d, SingleNodeDeploymentConfig):
            for side in (t.weight_broadcast, o.weight_broadcast):
                if hasattr(side, "inference_world_size") and world:
                    side.inference_world_size = world

    def _wire_replay_and_masks(self) -> None:
        t, o, i = self.trainer, self.orchestrator, self.inference
        if t.enable_router_replay:
            o.enable_return_routed_experts = True
            if i is not None:
                if i.router is not None and i.router.type == "llm-d":
                    raise ValueError("router replay needs the engines to return routed experts, which the llm-d "
                                     "router does not carry")
                i.vllm.enable_return_routed_experts = True
        if o.train.sampling.truncated and i is not None:
            i.enable_return_sampling_mask = True

    def _wire_inference_client(self) -> None:
        o, i, t = self.orchestrator, self.inference, self.trainer
        if i is None:
            return
        host = i.server.host if i.server.host not in (None, "0.0.0.0") else "localhost"
        base = f"http://{host}:{i.server.port}/v1"
        if o.model.client.base_url == "http://localhost:8000/v1":
            o.model.client.base_url = base
        if o.model.client.admin_base_url is None:
            o.model.client.admin_base_url = [base]
        if "model" not in i.vllm.model_fields_set:
            i.vllm.model = o.model.name

    @property
    def run_dir(self) -> Path:
        return self.output_dir / (self.run.dir or self.run.name)
