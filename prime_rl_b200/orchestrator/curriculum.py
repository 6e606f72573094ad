"""Curricula: which task a source launches next, and which finished groups are admitted
(reference: src/prime_rl/orchestrator/curriculum/*).

``StandardSampler``        round-robin over the task ids.
``DifficultyPoolSampler``  keeps a running solve rate per task and draws from the pools
                           ``easy`` / ``normal`` / ``hard`` (solve-rate thresholds, mixing
                           weights); unseen tasks count as ``normal``.
``AdvRangeGate``           rejects groups whose advantages all lie in ``[reject_min, reject_max]``
                           (no learning signal).
All samplers are checkpointable through ``state_dict`` / ``load_state_dict``.
"""

from __future__ import annotations

import random


class StandardSampler:
    def __init__(self, num_tasks: int, **_):
        self.num_tasks, self.next = max(1, num_tasks), 0

    def sample(self) -> int:
        t = self.next % self.num_tasks
        self.next += 1
        return t

    def update(self, task_id: int, mean_reward: float) -> None:
        pass

    def state_dict(self) -> dict:
        return {"next": self.next}

    def load_state_dict(self, sd: dict) -> None:
        self.next = int(sd.get("next", 0))


class DifficultyPoolSampler(StandardSampler):
    def __init__(self, num_tasks: int, pools: dict, seed: int = 42, ema: float = 0.5, **_):
        super().__init__(num_tasks)
        # pools sorted by threshold, hardest last: a task belongs to the first pool whose threshold it reaches
        self.pools = sorted(((n, float(p.threshold), float(p.weight)) for n, p in pools.items()), key=lambda x: -x[1])
        self.rng = random.Random(seed)
        self.ema = ema
        self.rate: dict[int, float] = {}

    def pool_of(self, task_id: int) -> str:
        r = self.rate.get(task_id)
        if r is None:
            return "normal" if any(n == "normal" for n, _, _ in self.pools) else self.pools[len(self.pools) // 2][0]
        for name, thr, _ in self.pools:
            if r >= thr:
                return name
        return self.pools[-1][0]

    def sample(self) -> int:
        names = [n for n, _, w in self.pools if w > 0]
        weights = [w for _, _, w in self.pools if w > 0]
        want = self.rng.choices(names, weights=weights, k=1)[0]
        # walk the round-robin pointer until a task of the wanted pool shows up (bounded)
        for _ in range(min(self.num_tasks, 256)):
            t = super().sample()
            if self.pool_of(t) == want:
                return t
        return super().sample()

    def update(self, task_id: int, mean_reward: float) -> None:
        old = self.rate.get(task_id)
        self.rate[task_id] = mean_reward if old is None else (1 - self.ema) * old + self.ema * mean_reward

    def state_dict(self) -> dict:
        return {"next": self.next, "rate": dict(self.rate), "rng": self.rng.getstate()}

    def load_state_dict(self, sd: dict) -> None:
        super().load_state_dict(sd)
        self.rate = {int(k): float(v) for k, v in sd.get("rate", {}).items()}
        if "rng" in sd:
            state = sd["rng"]
            self.rng.setstate((state[0], tuple(state[1]), state[2]))


class AdvRangeGate:
    def __init__(self, reject_min: float = 0.0, reject_max: float = 0.0, **_):
        self.reject_min, self.reject_max = reject_min, reject_max

    def admits(self, advantages: list[float]) -> bool:
        return not all(self.reject_min <= a <= self.reject_max for a in advantages)


def build_sampler(cfg, num_tasks: int):
    if cfg is None or cfg.sampler.type == "standard":
        return StandardSampler(num_tasks)
    return DifficultyPoolSampler(num_tasks, cfg.sampler.pools, seed=cfg.sampler.seed)
