"""Process identity and process-group bring-up: one process per GPU, ``torch.distributed``
over NCCL (gloo for CPU runs and tests)."""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class World:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    local_world_size: int = 1

    @property
    def is_master(self) -> bool:
        return self.rank == 0

    @property
    def num_nodes(self) -> int:
        return max(1, self.world_size // max(1, self.local_world_size))


_world: World | None = None


def get_world() -> World:
    global _world
    if _world is None:
        _world = World(
            rank=int(os.environ.get("RANK", 0)),
            world_size=int(os.environ.get("WORLD_SIZE", 1)),
            local_rank=int(os.environ.get("LOCAL_RANK", 0)),
            local_world_size=int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", 1))),
        )
    return _world


def reset_world() -> None:
    global _world
    _world = None


def setup_distributed(backend: str | None = None, timeout_seconds: int = 3600, device: str | None = None
                      ) -> torch.device:
    """Initialises the default process group when WORLD_SIZE > 1 and returns this rank's
    device. ``backend=None`` picks nccl on CUDA machines, gloo otherwise."""
    world = get_world()
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        dev = torch.device("cuda", world.local_rank % max(1, torch.cuda.device_count()))
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    if world.world_size > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "cpu:gloo,cuda:nccl" if use_cuda else "gloo"
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = dev
        dist.init_process_group(backend=backend, rank=world.rank, world_size=world.world_size,
                                timeout=datetime.timedelta(seconds=timeout_seconds), **kwargs)
    return dev


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def cleanup() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
