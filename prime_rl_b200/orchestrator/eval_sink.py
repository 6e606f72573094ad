"""Eval-side assembly: finished eval episodes are collected per (environment, eval step) epoch; an epoch is
complete once every expected rollout has either arrived, failed or been cancelled, and then yields one row
of metrics (mean reward, pass@k over the group, completion length, how many requests were lost).

Takes the place of the reference's ``EvalSink`` / ``EvalSource`` pair
(src/prime_rl/orchestrator/eval_sink.py:18-58, eval_source.py): evals are version-pinned measurements that
run through the same dispatcher as training rollouts, never go stale and never feed the trainer.
"""

from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field

from .types import Rollout


@dataclass
class EvalWork:
    """One eval example waiting to be dispatched ``group_size`` times."""

    source: object                 # orchestrator.Source
    task_id: int
    step: int


@dataclass
class _Epoch:
    expected: int
    group_size: int
    rewards: dict[int, list[float]] = field(default_factory=lambda: defaultdict(list))
    completion_tokens: int = 0
    arrived: int = 0
    failed: int = 0
    cancelled: int = 0
    version_min: int = 1 << 30
    version_max: int = -1

    @property
    def accounted(self) -> int:
        return self.arrived + self.failed + self.cancelled


class EvalSink:
    def __init__(self, pass_threshold: float = 1.0):
        self.epochs: dict[tuple[str, int], _Epoch] = {}
        self.pass_threshold = pass_threshold

    def expect(self, env_name: str, step: int, num_examples: int, group_size: int) -> None:
        self.epochs[(env_name, step)] = _Epoch(expected=num_examples * group_size, group_size=group_size)

    def add(self, r: Rollout, step: int) -> dict | None:
        ep = self.epochs.get((r.env_name, step))
        if ep is None:
            return None
        ep.rewards[r.task_id].append(r.reward)
        ep.completion_tokens += r.num_output_tokens
        ep.arrived += 1
        ep.version_min, ep.version_max = min(ep.version_min, r.policy_version), max(ep.version_max, r.policy_version)
        return self._maybe_finish(r.env_name, step)

    def fail(self, env_name: str, step: int, n: int = 1) -> dict | None:
        ep = self.epochs.get((env_name, step))
        if ep is None:
            return None
        ep.failed += n
        return self._maybe_finish(env_name, step)

    def cancel(self, env_name: str, step: int, n: int = 1) -> dict | None:
        ep = self.epochs.get((env_name, step))
        if ep is None:
            return None
        ep.cancelled += n
        return self._maybe_finish(env_name, step)

    def abandon(self, before_step: int) -> list[dict]:
        """Closes every epoch of an older step with what it has (a newer eval superseded it)."""
        out = []
        for env_name, step in [k for k in self.epochs if k[1] < before_step]:
            ep = self.epochs[(env_name, step)]
            ep.cancelled += max(0, ep.expected - ep.accounted)
            row = self._maybe_finish(env_name, step)
            if row is not None:
                out.append(row)
        return out

    def _maybe_finish(self, env_name: str, step: int) -> dict | None:
        ep = self.epochs[(env_name, step)]
        if ep.accounted < ep.expected:
            return None
        del self.epochs[(env_name, step)]
        rewards = [x for rs in ep.rewards.values() for x in rs]
        n = max(1, len(rewards))
        solved = sum(any(x >= self.pass_threshold for x in rs) for rs in ep.rewards.values())
        return {"env": env_name, "step": step, "num_examples": len(ep.rewards), "group_size": ep.group_size,
                "reward/mean": sum(rewards) / n, f"pass@{ep.group_size}": solved / max(1, len(ep.rewards)),
                "completion_len/mean": ep.completion_tokens / n, "rollouts": ep.arrived, "failed": ep.failed,
                "cancelled": ep.cancelled,
                "policy_version": ep.version_max if ep.version_max >= 0 else step}
