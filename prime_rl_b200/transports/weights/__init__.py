"""Trainer -> inference weight transports.

All transports share one handshake through marker files in
``<run_dir>/broadcasts/step_N/`` (reference: src/prime_rl/transports/weights/base.py:17-93):

    trainer master: mkdir, touch .sender_ready, wait (<= timeout) for .receiver_ready,
                    touch .started, transfer, touch .finished, drop dirs older than step-1
    receiver      : sees .sender_ready, pauses the engine, touch .receiver_ready,
                    takes part in / waits for the transfer, applies the weights, resumes

filesystem  HF safetensors shards (or a PEFT adapter directory for LoRA runs) in the step dir;
nccl        layer-by-layer broadcast from trainer rank 0 to every engine GPU (baseline);
p2p         the trainer pushes its shards straight into the engine's weight buffers over
            NVLink peer memory, quantising to block-scaled fp8 on the way (same box).
"""

from __future__ import annotations

import shutil
import time
from pathlib import Path

import torch.distributed as dist

from ...utils.logger import get_logger
from ...utils.pathing import get_broadcast_dir, get_step_path, list_steps

def _null():
    import contextlib

    return contextlib.nullcontext()


SENDER_READY, RECEIVER_READY, STARTED, FINISHED = ".sender_ready", ".receiver_ready", ".started", ".finished"


class WeightSender:
    def __init__(self, config, run_dir: Path, world, require_ack: bool = True):
        self.config, self.world = config, world
        self.dir = get_broadcast_dir(run_dir)
        self.require_ack = require_ack
        self.logger = get_logger()

    def step_dir(self, step: int) -> Path:
        return get_step_path(self.dir, step)

    def _wait(self, path: Path, what: str) -> None:
        t0 = time.monotonic()
        while not path.exists():
            if time.monotonic() - t0 > self.config.timeout:
                raise TimeoutError(f"weight broadcast: no {what} within {self.config.timeout}s ({path})")
            time.sleep(0.02)

    def broadcast(self, model, step: int) -> None:
        d = self.step_dir(step)
        if self.world.is_master:
            d.mkdir(parents=True, exist_ok=True)
            (d / SENDER_READY).touch()
            if self.require_ack:
                self._wait(d / RECEIVER_READY, "receiver acknowledgement")
            (d / STARTED).touch()
        if dist.is_initialized():
            dist.barrier()
        with model.full_parameters() if hasattr(model, "full_parameters") else _null():
            self._broadcast(model, step, d)       # sharded parameters are whole for the duration
        if dist.is_initialized():
            dist.barrier()
        if self.world.is_master:
            (d / FINISHED).touch()
            for s in list_steps(self.dir):
                if s < step - 1:
                    shutil.rmtree(self.step_dir(s), ignore_errors=True)

    def _broadcast(self, model, step: int, d: Path) -> None:
        raise NotImplementedError


class FileSystemWeightSender(WeightSender):
    """The consumer only needs the finished directory, so the sender does not wait for an
    acknowledgement before writing."""

    def __init__(self, config, run_dir, world, lora_cfg=None):
        super().__init__(config, run_dir, world, require_ack=False)
        self.lora_cfg = lora_cfg

    def _broadcast(self, model, step, d):
        from ...trainer.weights import save_hf_checkpoint, save_lora_adapter

        from ...models.convert import expert_parallel_info

        if expert_parallel_info(model) is not None and self.lora_cfg is None:
            save_hf_checkpoint(model, d)        # collective: every ep rank writes the experts it owns
            return
        if not self.world.is_master:
            return  # replicated weights: one writer is enough
        if self.lora_cfg is not None:
            save_lora_adapter(model, d, self.lora_cfg.rank, self.lora_cfg.alpha, self.lora_cfg.target_modules)
        else:
            save_hf_checkpoint(model, d)


class WeightReceiver:
    """Orchestrator-side half of the handshake. ``engine`` is an admin client with
    ``pause()``, ``resume()`` and ``update_weights(weight_dir | None)``."""

    def __init__(self, config, run_dir: Path, engine):
        self.config, self.engine = config, engine
        self.dir = get_broadcast_dir(run_dir)

    def pending_step(self, after: int) -> int | None:
        for s in list_steps(self.dir):
            if s > after and (get_step_path(self.dir, s) / SENDER_READY).exists():
                return s
        return None

    async def receive(self, step: int) -> None:
        import asyncio

        d = get_step_path(self.dir, step)
        in_memory = self.config.type != "filesystem"
        if in_memory:
            await self.engine.pause()
            (d / RECEIVER_READY).touch()
            await self.engine.update_weights(None)      # workers join the collective
        else:
            (d / RECEIVER_READY).touch()
            t0 = time.monotonic()
            while not (d / FINISHED).exists():
                if time.monotonic() - t0 > self.config.timeout:
                    raise TimeoutError(f"weights for step {step} not finished after {self.config.timeout}s")
                await asyncio.sleep(0.05)
            await self.engine.pause()
            await self.engine.update_weights(str(d))
        await self.engine.resume()


def setup_weight_sender(config, run_dir: Path, world, model, lora: bool = False, lora_cfg=None):
    if config.type == "filesystem":
        return FileSystemWeightSender(config, run_dir, world, lora_cfg=lora_cfg if lora else None)
    if config.type == "nccl":
        from .nccl import NCCLWeightSender

        sender = NCCLWeightSender(config, run_dir, world)
        sender.connect_in_background(next(model.parameters()).device)     # the engines join before the first batch
        return sender
    if config.type == "p2p":
        from .p2p import P2PWeightSender

        return P2PWeightSender(config, run_dir, world)
    raise ValueError(f"weight broadcast type '{config.type}' is not available in this build")
