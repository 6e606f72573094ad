"""Per-token trainer annotations: for every rollout branch that carries a trace id, the
trainer's own log-probabilities and entropies of its tokens, written next to the rollout trace
so that a viewer can overlay "what the trainer saw" on "what the engine sampled".

Records are collected per micro-batch on every rank, gathered to rank 0 once per step and
handed to the monitors' ``log_annotations`` (stream ``"trainer"``). Same role as the reference's
``AnnotationWriter`` (src/prime_rl/trainer/rl/annotations.py:1-90).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class AnnotationWriter:
    def __init__(self, monitor, rank: int = 0, world_size: int = 1, group=None):
        self.monitor, self.rank, self.world_size, self.group = monitor, rank, world_size, group
        self._pending: list[dict] = []

    def collect(self, mb, logprobs: torch.Tensor, entropy: torch.Tensor, step: int) -> None:
        """``mb``: the micro-batch (``sequence_lengths``, ``trace_ids``, ``branch_indices``,
        ``loss_mask``); ``logprobs`` / ``entropy``: fp32 ``[T]`` aligned with ``mb.input_ids``."""
        if not getattr(mb, "trace_ids", None):
            return
        lp = logprobs.detach().float().cpu()
        en = entropy.detach().float().cpu()
        mask = mb.loss_mask.detach().cpu()
        t0 = 0
        for n, trace_id, branch in zip(mb.sequence_lengths, mb.trace_ids, mb.branch_indices or []):
            if trace_id:
                self._pending.append({
                    "trace_id": trace_id, "branch_index": int(branch), "step": int(step),
                    "logprobs": [round(float(x), 6) for x in lp[t0:t0 + n]],
                    "entropy": [round(float(x), 6) for x in en[t0:t0 + n]],
                    "loss_mask": [bool(x) for x in mask[t0:t0 + n]],
                })
            t0 += n

    def flush(self) -> int:
        """Gathers this step's records on rank 0 and writes them; returns how many were written."""
        mine, self._pending = self._pending, []
        records = mine
        if self.world_size > 1 and dist.is_initialized():
            gathered = [None] * self.world_size if self.rank == 0 else None
            dist.gather_object(mine, gathered, dst=0, group=self.group)
            records = [r for part in (gathered or []) for r in part]
        if self.rank == 0 and records:
            self.monitor.log_annotations(records, "trainer")
            return len(records)
        return 0
