"""Adaptive in-flight concurrency (AIMD on the engines' KV-cache usage).

Grow x1.25 per turnover while usage < 0.6; hold between 0.6 and 0.8 (target 0.7); soft-trim
above 0.8; hard-trim (and ask the dispatcher to cancel the newest episodes) above 0.9; cut on
preemptions or a growing wait queue (reference: src/prime_rl/orchestrator/concurrency.py:41-90).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ConcurrencyDecision:
    limit: int
    cancel: int = 0
    reason: str = "hold"


class ConcurrencyController:
    GROW_BELOW, SOFT_TRIM_ABOVE, HARD_TRIM_ABOVE, TARGET = 0.6, 0.8, 0.9, 0.7

    def __init__(self, config, group_size: int = 1):
        self.min = max(config.min_inflight, 1)
        self.max = config.max_inflight
        self.limit = config.initial_inflight or max(self.min, 4 * group_size)
        self.limit = self._clamp(self.limit)
        self.last_preemptions = 0.0
        self.completed_since_update = 0

    def _clamp(self, v: int) -> int:
        v = max(self.min, int(v))
        return min(v, self.max) if self.max is not None else v

    def on_episode_done(self) -> None:
        self.completed_since_update += 1

    def update(self, kv_usage: float, waiting: float = 0.0, preemptions_total: float = 0.0, inflight: int = 0
               ) -> ConcurrencyDecision:
        new_preempt = preemptions_total - self.last_preemptions
        self.last_preemptions = preemptions_total
        old = self.limit
        cancel, reason = 0, "hold"
        if kv_usage > self.HARD_TRIM_ABOVE or new_preempt > 0:
            self.limit = self._clamp(min(self.limit, max(inflight, 1)) * 0.75)
            cancel = max(0, inflight - self.limit)
            reason = "hard_trim"
        elif kv_usage > self.SOFT_TRIM_ABOVE or waiting > 0.25 * max(inflight, 1):
            self.limit = self._clamp(self.limit * self.TARGET / max(kv_usage, self.TARGET))
            reason = "soft_trim"
        elif kv_usage < self.GROW_BELOW and self.completed_since_update >= max(1, old // 2) and inflight >= old * 0.9:
            self.limit = self._clamp(max(old + 1, old * 1.25))
            reason = "grow"
        if reason != "hold":
            self.completed_since_update = 0
        return ConcurrencyDecision(self.limit, cancel, reason)
