"""Micro-batch transports between the orchestrator and the trainer ranks.

filesystem  ``<run_dir>/batches/step_N/rank_R.bin`` written to ``.tmp`` then renamed;
zmq         sender binds PUB on ``port`` and PULL on ``port + 1``, waits for one READY per data
            rank, then publishes ``[b"data_rank|R|", payload]``; receivers SUB to their topic.
(reference: src/prime_rl/transports/batch/{filesystem,zmq}.py)
"""

from __future__ import annotations

import time
from pathlib import Path

import torch

from ...utils.pathing import get_batch_dir, get_step_path
from .types import (MicroBatch, RoutedExperts, SamplingMask, TrainingSample, decode_micro_batches,  # noqa: F401
                    decode_routed_experts, decode_sampling_mask, decode_tensor, encode_micro_batches,
                    encode_tensor)


def micro_batch_to_tensors(mb: MicroBatch):
    from ...trainer.data import TensorMicroBatch

    T = len(mb.input_ids)
    f32 = lambda x: torch.tensor(x, dtype=torch.float32) if x is not None else None  # noqa: E731
    return TensorMicroBatch(
        input_ids=torch.tensor(mb.input_ids, dtype=torch.long),
        position_ids=torch.tensor(mb.position_ids, dtype=torch.int32),
        advantages=f32(mb.advantages), inference_logprobs=f32(mb.inference_logprobs),
        loss_mask=torch.tensor(mb.loss_mask, dtype=torch.bool), temperatures=f32(mb.temperatures),
        sequence_lengths=list(mb.sequence_lengths), env_names=list(mb.env_names), ref_logprobs=f32(mb.ref_logprobs),
        routed_experts=decode_routed_experts(mb.routed_experts) if mb.routed_experts is not None else None,
        sampling_mask=decode_sampling_mask(mb.sampling_mask, T) if mb.sampling_mask is not None else None,
        rl_weights=f32(mb.rl_weights), ce_weights=f32(mb.ce_weights), ref_kl_weights=f32(mb.ref_kl_weights),
        trace_ids=mb.trace_ids, branch_indices=mb.branch_indices,
        mm_kwargs={k: decode_tensor(e) for k, e in mb.mm_kwargs.items()} if mb.mm_kwargs else None,
        mm_token_type_ids=torch.tensor(mb.mm_token_type_ids, dtype=torch.int32) if mb.mm_token_type_ids else None,
        lora_num_tokens=torch.tensor([T], dtype=torch.int32))


class FileSystemBatchSender:
    def __init__(self, run_dir: Path):
        self.dir = get_batch_dir(run_dir)

    def send(self, step: int, grid: list[list[MicroBatch]]) -> None:
        """grid[dp_rank][micro_step]"""
        d = get_step_path(self.dir, step)
        d.mkdir(parents=True, exist_ok=True)
        for rank, mbs in enumerate(grid):
            tmp = d / f"rank_{rank}.bin.tmp"
            tmp.write_bytes(encode_micro_batches(mbs))
            tmp.replace(d / f"rank_{rank}.bin")

    def close(self) -> None:
        pass


class FileSystemBatchReceiver:
    def __init__(self, run_dir: Path, dp_rank: int, start_step: int, poll: float = 0.05,
                 timeout: float | None = None):
        self.dir, self.rank, self.step, self.poll, self.timeout = get_batch_dir(run_dir), dp_rank, start_step, poll, timeout

    def _path(self) -> Path:
        return get_step_path(self.dir, self.step) / f"rank_{self.rank}.bin"

    def wait(self) -> None:
        t0 = time.monotonic()
        while not self._path().exists():
            if self.timeout is not None and time.monotonic() - t0 > self.timeout:
                raise TimeoutError(f"no batch for step {self.step} rank {self.rank} after {self.timeout}s")
            time.sleep(self.poll)

    def receive(self) -> list[MicroBatch]:
        self.wait()
        out = decode_micro_batches(self._path().read_bytes())
        self.step += 1
        return out

    def close(self) -> None:
        pass


class ZMQBatchSender:
    def __init__(self, config, num_ranks: int, ready_timeout: float = 600.0):
        import zmq

        self.ctx = zmq.Context.instance()
        self.pub = self.ctx.socket(zmq.PUB)
        self.pub.setsockopt(zmq.SNDHWM, config.hwm)
        self.pub.bind(f"tcp://*:{config.port}")
        self.pull = self.ctx.socket(zmq.PULL)
        self.pull.bind(f"tcp://*:{config.port + 1}")
        self.num_ranks, self.ready, self.ready_timeout = num_ranks, set(), ready_timeout

    def wait_ready(self) -> None:
        import zmq

        deadline = time.monotonic() + self.ready_timeout
        while len(self.ready) < self.num_ranks:
            left = deadline - time.monotonic()
            if left <= 0:
                raise TimeoutError(f"only {len(self.ready)}/{self.num_ranks} trainer ranks reported READY")
            if self.pull.poll(int(min(left, 1.0) * 1000), zmq.POLLIN):
                msg = self.pull.recv()
                if msg.startswith(b"READY|"):
                    self.ready.add(int(msg.split(b"|")[1]))

    def send(self, step: int, grid: list[list[MicroBatch]]) -> None:
        self.wait_ready()
        for rank, mbs in enumerate(grid):
            self.pub.send_multipart([f"data_rank|{rank}|".encode(), encode_micro_batches(mbs)])

    def close(self) -> None:
        self.pub.close(0)
        self.pull.close(0)


class ZMQBatchReceiver:
    def __init__(self, config, dp_rank: int):
        import zmq

        self.ctx = zmq.Context.instance()
        self.sub = self.ctx.socket(zmq.SUB)
        self.sub.setsockopt(zmq.RCVHWM, config.hwm)
        self.sub.connect(f"tcp://{config.host}:{config.port}")
        self.sub.setsockopt(zmq.SUBSCRIBE, f"data_rank|{dp_rank}|".encode())
        self.push = self.ctx.socket(zmq.PUSH)
        self.push.connect(f"tcp://{config.host}:{config.port + 1}")
        self.rank = dp_rank
        self._pending: bytes | None = None
        time.sleep(0.2)  # let the subscription propagate before announcing readiness
        self.push.send(f"READY|{dp_rank}".encode())

    def wait(self) -> None:
        if self._pending is None:
            _, payload = self.sub.recv_multipart()
            self._pending = payload

    def receive(self) -> list[MicroBatch]:
        self.wait()
        payload, self._pending = self._pending, None
        return decode_micro_batches(payload)

    def close(self) -> None:
        self.sub.close(0)
        self.push.close(0)


def setup_batch_sender(run_dir: Path, num_ranks: int, config):
    if config.type == "zmq":
        return ZMQBatchSender(config, num_ranks)
    return FileSystemBatchSender(run_dir)


def setup_batch_receiver(run_dir: Path, dp_rank: int, start_step: int, config):
    if config.type == "zmq":
        return ZMQBatchReceiver(config, dp_rank)
    return FileSystemBatchReceiver(run_dir, dp_rank, start_step)
