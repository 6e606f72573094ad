"""Micro-batch containers and the trainer-side data loaders.

A micro-batch is one packed row of tokens (``[T]`` tensors plus document lengths). Tensors
are created in pinned host memory so that the per-step host->device copies are asynchronous.
``FakeDataLoader`` mirrors the reference's seeded synthetic loader
(src/prime_rl/trainer/rl/data.py:66-175): the seed depends on the data-parallel rank only,
so that all context-parallel ranks of one replica see the same rows.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path

import torch


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except RuntimeError:
            return t
    return t


@dataclass
class TensorMicroBatch:
    input_ids: torch.Tensor                  # int64 [T]
    position_ids: torch.Tensor               # int32 [T]
    advantages: torch.Tensor                 # fp32 [T]
    inference_logprobs: torch.Tensor         # fp32 [T]
    loss_mask: torch.Tensor                  # bool [T]
    temperatures: torch.Tensor               # fp32 [T]
    sequence_lengths: list[int]
    env_names: list[str] = field(default_factory=list)
    ref_logprobs: torch.Tensor | None = None
    routed_experts: torch.Tensor | None = None     # int [T, layers, k]
    sampling_mask: torch.Tensor | None = None      # int32 [T, K], -1 padded
    rl_weights: torch.Tensor | None = None
    ce_weights: torch.Tensor | None = None
    ref_kl_weights: torch.Tensor | None = None
    trace_ids: list[str] | None = None
    branch_indices: list[int] | None = None
    lora_num_tokens: torch.Tensor | None = None
    mm_kwargs: dict | None = None                  # image tensors of the row: pixel_values, image_grid_thw
    mm_token_type_ids: torch.Tensor | None = None  # int32 [T]: 0 text, 1 image placeholder

    TENSOR_FIELDS = ("input_ids", "position_ids", "advantages", "inference_logprobs", "loss_mask", "temperatures",
                     "ref_logprobs", "routed_experts", "sampling_mask", "rl_weights", "ce_weights",
                     "ref_kl_weights")

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.numel())

    def pin(self) -> "TensorMicroBatch":
        for f in self.TENSOR_FIELDS:
            t = getattr(self, f)
            if t is not None:
                setattr(self, f, _pin(t))
        return self

    def to(self, device, non_blocking: bool = True) -> "TensorMicroBatch":
        kw = {f: (getattr(self, f).to(device, non_blocking=non_blocking) if getattr(self, f) is not None else None)
              for f in self.TENSOR_FIELDS}
        return TensorMicroBatch(sequence_lengths=self.sequence_lengths, env_names=self.env_names,
                                trace_ids=self.trace_ids, branch_indices=self.branch_indices,
                                lora_num_tokens=self.lora_num_tokens,
                                mm_kwargs={k: v.to(device, non_blocking=non_blocking) for k, v in self.mm_kwargs.items()}
                                if self.mm_kwargs else None,
                                mm_token_type_ids=self.mm_token_type_ids, **kw)

    def h2d_bytes(self) -> int:
        return sum(getattr(self, f).numel() * getattr(self, f).element_size()
                   for f in self.TENSOR_FIELDS if getattr(self, f) is not None)

    def loss_token_counts(self) -> tuple[int, int, int]:
        """(rl, ce, ref_kl) token counts of this micro-batch, the denominators' local parts."""
        mask = self.loss_mask
        rl = int((mask & (self.rl_weights != 0)).sum()) if self.rl_weights is not None else int(mask.sum())
        ce = int((self.ce_weights != 0).sum()) if self.ce_weights is not None else 0
        rk = int((self.ref_kl_weights != 0).sum()) if self.ref_kl_weights is not None else 0
        return rl, ce, rk


class FakeDataLoader:
    """Seeded synthetic micro-batches of ``seq_len`` tokens; ``batch_size`` is the global
    number of micro-batches per step (split over data-parallel ranks)."""

    def __init__(self, batch_size: int, seq_len: int, dp_world_size: int, dp_rank: int, *,
                 generate_samples: bool = False, vocab_size: int = 100, docs_per_batch: int = 1,
                 prompt_fraction: float = 0.0, pin: bool = True):
        self.num_micro_batches = max(1, batch_size // dp_world_size)
        self.seq_len, self.dp_rank = seq_len, dp_rank
        self.generate_samples, self.vocab_size = generate_samples, vocab_size
        self.docs_per_batch, self.prompt_fraction, self.pin = docs_per_batch, prompt_fraction, pin
        self.batch_counter = 0

    def wait_for_batch(self) -> None:
        return

    def get_batch(self) -> list[TensorMicroBatch]:
        out = []
        for i in range(self.num_micro_batches):
            seed = self.dp_rank * 1_000_000 + self.batch_counter * 1000 + i
            gen = torch.Generator().manual_seed(seed)
            mb = self._sample(gen) if self.generate_samples else self._uniform(gen)
            out.append(mb.pin() if self.pin else mb)
        self.batch_counter += 1
        return out

    def state_dict(self) -> dict:
        return {"batch_counter": self.batch_counter}

    def load_state_dict(self, sd: dict) -> None:
        self.batch_counter = sd.get("batch_counter", 0)

    def _make(self, lengths: list[int], gen: torch.Generator) -> TensorMicroBatch:
        T = sum(lengths)
        ids = torch.randint(0, self.vocab_size, (T,), generator=gen)
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths])
        mask = torch.ones(T, dtype=torch.bool)
        if self.prompt_fraction > 0:
            start = 0
            for n in lengths:
                mask[start:start + int(n * self.prompt_fraction)] = False
                start += n
        return TensorMicroBatch(
            input_ids=ids, position_ids=pos, advantages=torch.randn(T, generator=gen),
            inference_logprobs=-torch.rand(T, generator=gen) * 2.0 - 0.05, loss_mask=mask,
            temperatures=torch.ones(T), sequence_lengths=lengths, env_names=["fake"] * len(lengths),
            lora_num_tokens=torch.tensor([T], dtype=torch.int32))

    def _uniform(self, gen) -> TensorMicroBatch:
        d = self.docs_per_batch
        base = self.seq_len // d
        lengths = [base] * (d - 1) + [self.seq_len - base * (d - 1)]
        return self._make(lengths, gen)

    def _sample(self, gen) -> TensorMicroBatch:
        lengths, total = [], 0
        while total < self.seq_len:
            n = int(torch.randint(1, max(2, self.seq_len // 8), (1,), generator=gen))
            n = min(n, self.seq_len - total)
            lengths.append(n)
            total += n
        return self._make(lengths, gen)


class DataLoader:
    """Receives packed micro-batches from the orchestrator (one stream per data-parallel
    rank) and turns them into tensors."""

    def __init__(self, output_dir: Path, start_step: int, dp_world_size: int, dp_rank: int, transport_config):
        from ..transports.batch import setup_batch_receiver

        self.receiver = setup_batch_receiver(output_dir, dp_rank, start_step, transport_config)

    def wait_for_batch(self) -> None:
        self.receiver.wait()

    def get_batch(self) -> list[TensorMicroBatch]:
        from ..transports.batch import micro_batch_to_tensors

        return [micro_batch_to_tensors(mb).pin() for mb in self.receiver.receive()]
