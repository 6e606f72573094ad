"""Trainer checkpoints in torch DCP format.

Layout ``<run_dir>/checkpoints/step_N/trainer/`` holding the DCP shards of
``{"app": {"model", "optimizer", "progress"}}`` with model tensors under their *prime*
names (per-projection, experts stacked), which is what the reference writes
(src/prime_rl/trainer/ckpt.py:48-213) — runtime fusions never reach a checkpoint.
Optimizer state is keyed by the same names. ``dataloader/rank_R.pt`` is written per rank.
Retention follows ``keep_last`` / ``keep_interval``; only the master rank deletes.
"""

from __future__ import annotations

import json

import shutil
from dataclasses import asdict, dataclass
from pathlib import Path

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ..models import convert
from ..utils.logger import get_logger
from ..utils.pathing import get_ckpt_dir, get_step_path, latest_step, list_steps


@dataclass
class Progress:
    step: int = 0
    total_tokens: int = 0
    total_samples: int = 0


def _optimizer_state_prime(sd: dict, arch) -> dict:
    """``FlatOptimizer.state_dict()`` tensors under prime names (fused parameters split like the weights)."""
    out = {"step": torch.tensor(sd["step"])}
    for key, named in sd["state"].items():
        out[key] = convert.native_to_prime(dict(named), arch)
    return out


def _ep_mesh(info, device_type: str):
    """Device mesh ``(replica, ep)`` (or just ``(ep,)``) over which expert-sharded tensors are
    described to DCP. Creating it is a collective over all ranks; it is cached on the record."""
    if "mesh" not in info:
        from torch.distributed.device_mesh import DeviceMesh

        lists = info["rank_lists"]
        if len(lists) == 1:
            info["mesh"] = DeviceMesh.from_group(info["group"], device_type, mesh=torch.tensor(lists[0]),
                                                 mesh_dim_names=("ep",))
        else:
            info["mesh"] = DeviceMesh(device_type, torch.tensor(lists), mesh_dim_names=("ep_replica", "ep"))
    return info["mesh"]


def _describe_expert_shards(tree: dict, model) -> dict:
    """Expert-parallel ranks keep ``[E / ep, ...]`` slices under the same names. DCP treats equal names
    of plain tensors as replicas and would keep one rank's slice, so the slices are presented as
    DTensors sharded on dim 0 over the ep group (replicated over the groups that hold the same
    slice): the checkpoint then holds the full ``[E, ...]`` stacks and can be read back with another
    ep degree. The wrappers share storage with the live tensors, so a load still lands in place."""
    info = convert.expert_parallel_info(model)
    if info is None:
        return tree
    from torch.distributed.tensor import DTensor, Replicate, Shard

    def wrap(prefix: str, node):
        if isinstance(node, dict):
            return {k: wrap(f"{prefix}.{k}", v) for k, v in node.items()}
        if isinstance(node, torch.Tensor) and convert.is_expert_sharded_key(prefix) and node.dim() >= 1 \
                and node.shape[0] == info["local_experts"]:
            mesh = _ep_mesh(info, node.device.type)
            placements = [Shard(0)] if mesh.ndim == 1 else [Replicate(), Shard(0)]
            return DTensor.from_local(node.detach(), mesh, placements, run_check=False)
        return node

    return wrap("", tree)


class CheckpointManager:
    def __init__(self, run_dir: Path, config, *, is_master: bool = True, rank: int = 0):
        self.run_dir, self.config, self.is_master, self.rank = run_dir, config, is_master, rank
        self.ckpt_dir = get_ckpt_dir(Path(config.output_dir) if config and config.output_dir else run_dir)
        self.saved_steps: list[int] = list_steps(self.ckpt_dir)

    def step_path(self, step: int) -> Path:
        return get_step_path(self.ckpt_dir, step) / "trainer"

    def latest(self) -> int | None:
        return latest_step(self.ckpt_dir)

    # ------------------------------------------------------------------ save
    def save(self, step: int, model, optimizer, progress: Progress, dataloader=None) -> Path:
        path = self.step_path(step)
        if self.is_master:
            path.mkdir(parents=True, exist_ok=True)
        if dist.is_initialized():
            dist.barrier()
        with model.full_parameters():          # sharded parameters are whole while the checkpoint is written
            app = {"model": convert.model_state(model, "prime", include_lora=True)}
            if not (self.config and self.config.skip_optimizer) and optimizer is not None:
                app["optimizer"] = _optimizer_state_prime(optimizer.state_dict(), model.arch)
            app = _describe_expert_shards(app, model)
            if not (self.config and self.config.skip_progress):
                app["progress"] = {k: torch.tensor(v) for k, v in asdict(progress).items()}
            dcp.save({"app": app}, checkpoint_id=str(path))
        if dist.is_initialized():
            dist.barrier()
        if self.is_master:
            # sizes of the shard files: a truncated copy must fail loudly at load time
            sizes = {f.name: f.stat().st_size for f in path.glob("*.distcp")}
            tmp = path / "sizes.json.tmp"
            tmp.write_text(json.dumps(sizes))
            tmp.replace(path / "sizes.json")
        if dataloader is not None and hasattr(dataloader, "state_dict") and \
                not (self.config and self.config.skip_dataloader):
            dl = path / "dataloader"
            dl.mkdir(parents=True, exist_ok=True)
            torch.save(dataloader.state_dict(), dl / f"rank_{self.rank}.pt")
        if dist.is_initialized():
            dist.barrier()
        if step not in self.saved_steps:
            self.saved_steps.append(step)
        get_logger().info(f"saved checkpoint step {step} to {path}")
        return path

    # ------------------------------------------------------------------ load
    def load(self, step: int, model, optimizer, progress: Progress, dataloader=None, path: Path | None = None) -> None:
        path = path or self.step_path(step)
        if not path.exists():
            raise FileNotFoundError(f"checkpoint not found: {path}")
        sizes_file = path / "sizes.json"
        if sizes_file.exists():
            for name, size in json.loads(sizes_file.read_text()).items():
                f = path / name
                if not f.exists() or f.stat().st_size != size:
                    have = f.stat().st_size if f.exists() else "missing"
                    raise RuntimeError(f"checkpoint shard {f} is damaged: {have} bytes, expected {size}")
        has_opt = optimizer is not None and not (self.config and self.config.skip_optimizer)
        opt_sd = None
        with model.full_parameters(writeback=True):      # sharded parameters: load whole, keep the own slices
            app = {"model": convert.model_state(model, "prime", include_lora=True)}
            if has_opt:
                opt_sd = optimizer.state_dict()
                app["optimizer"] = _optimizer_state_prime(opt_sd, model.arch)
            app = _describe_expert_shards(app, model)
            if not (self.config and self.config.skip_progress):
                app["progress"] = {k: torch.tensor(v) for k, v in asdict(progress).items()}
            dcp.load({"app": app}, checkpoint_id=str(path))
        # The prime-layout model tensors are views of the live parameters, so the load landed in place.
        # Optimizer tensors are views of ``opt_sd``: the live buffers where the state is not partitioned,
        # gathered full-length copies where it is (ZeRO). ``load_state_dict`` copies them back into the
        # owner's slice, refreshes the fp32 master and re-derives the compute-dtype parameters from it.
        if has_opt:
            opt_sd["step"] = int(app["optimizer"]["step"])
            optimizer.load_state_dict(opt_sd)
        if "progress" in app:
            for k, v in app["progress"].items():
                setattr(progress, k, int(v))
        dl = path / "dataloader" / f"rank_{self.rank}.pt"
        if dataloader is not None and dl.exists() and hasattr(dataloader, "load_state_dict"):
            dataloader.load_state_dict(torch.load(dl))
        get_logger().info(f"loaded checkpoint {path}")

    # ------------------------------------------------------------------ retention
    def maybe_clean(self) -> None:
        if not self.is_master or self.config is None:
            return
        keep_last, keep_interval = self.config.keep_last, self.config.keep_interval
        if keep_last is None:
            return
        steps = sorted(self.saved_steps)
        doomed = steps[:-keep_last] if keep_last else []
        for s in doomed:
            if keep_interval and s % keep_interval == 0:
                continue
            shutil.rmtree(get_step_path(self.ckpt_dir, s), ignore_errors=True)
            self.saved_steps.remove(s)
