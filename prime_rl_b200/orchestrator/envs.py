"""Environments: a task source plus an episode runner that talks to the inference pool.

The reference delegates this to ``verifiers`` environments behind env-server processes
(src/prime_rl/orchestrator/envs.py:69-231). Here the protocol is self-contained:

    class Environment:
        async def rollout(client, task, sampling, policy_version, group_id) -> Rollout

Built-in token-level environments need no tokenizer or dataset (there is no network):

``reverse-text``  reward = longest-common-subsequence ratio between the completion and the
                  reversed prompt payload (the shape of the reference's CI task);
``copy``          reward for repeating the payload;
``count-up``      multi-turn: the environment appends an observation token after each turn.
"""

from __future__ import annotations

import importlib
import random
from typing import Any

from .types import Rollout, Turn


def lcs_ratio(a: list[int], b: list[int]) -> float:
    if not a or not b:
        return 0.0
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b):
            cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
        prev = cur
    return 2.0 * prev[-1] / (len(a) + len(b))


class Environment:
    name = "env"

    def __init__(self, name: str | None = None, vocab_size: int = 4096, seed: int = 0, num_tasks: int = 4096, **_):
        self.name = name or self.name
        self.vocab_size, self.seed, self.num_tasks = vocab_size, seed, num_tasks

    def task(self, task_id: int) -> dict[str, Any]:
        raise NotImplementedError

    def score(self, task: dict[str, Any], completion: list[int]) -> float:
        raise NotImplementedError

    async def rollout(self, client, task_id: int, sampling, policy_version: int, group_id: str) -> Rollout:
        task = self.task(task_id)
        out = await client.generate(task["prompt"], sampling, cache_salt=str(policy_version))
        turn = Turn(task["prompt"], out["token_ids"], out["logprobs"], temperature=sampling.temperature,
                    routed_experts=out.get("routed_experts"), sampling_mask=out.get("sampling_mask"),
                    finish_reason=out.get("finish_reason"))
        reward = self.score(task, out["token_ids"])
        return Rollout(env_name=self.name, task_id=task_id, group_id=group_id, turns=[turn], reward=reward,
                       policy_version=out.get("policy_version", policy_version), metrics={"reward": reward})


class ReverseTextEnv(Environment):
    name = "reverse-text"

    def __init__(self, min_len: int = 4, max_len: int = 12, **kw):
        super().__init__(**kw)
        self.min_len, self.max_len = min_len, max_len

    def task(self, task_id: int):
        rng = random.Random(self.seed * 1_000_003 + task_id)
        n = rng.randint(self.min_len, self.max_len)
        payload = [rng.randrange(4, self.vocab_size) for _ in range(n)]
        return {"prompt": [1] + payload + [2], "payload": payload, "max_tokens": n}

    def score(self, task, completion):
        return lcs_ratio(completion[: len(task["payload"])], task["payload"][::-1])


class CopyEnv(ReverseTextEnv):
    name = "copy"

    def score(self, task, completion):
        return lcs_ratio(completion[: len(task["payload"])], task["payload"])


class LowTokenEnv(ReverseTextEnv):
    """Dense, quickly learnable reward for runs from random weights (where no pretrained model can be had): the
    fraction of completion tokens whose id lies in the lowest eighth of the vocabulary. A random policy starts near
    0.125 and a working trainer / weight-sync loop raises it within tens of steps."""

    name = "low-token"

    def score(self, task, completion):
        if not completion:
            return 0.0
        cut = max(1, self.vocab_size // 8)
        return sum(1 for t in completion if t < cut) / len(completion)


class CountUpEnv(Environment):
    """Two-turn episode: after the first completion the environment appends an observation
    token; reward counts completions that start with the token following the observation."""

    name = "count-up"

    def task(self, task_id: int):
        rng = random.Random(self.seed * 7919 + task_id)
        start = rng.randrange(4, self.vocab_size - 8)
        return {"prompt": [1, start, 2], "start": start}

    def score(self, task, completion):
        return 1.0 if completion and completion[0] == task["start"] + 1 else 0.0

    async def rollout(self, client, task_id, sampling, policy_version, group_id):
        task = self.task(task_id)
        turns, prompt, reward = [], list(task["prompt"]), 0.0
        for step in range(2):
            out = await client.generate(prompt, sampling, cache_salt=str(policy_version))
            turns.append(Turn(list(prompt), out["token_ids"], out["logprobs"], temperature=sampling.temperature,
                              finish_reason=out.get("finish_reason"),
                              role_spans=[("user", 0, len(task["prompt"]))] +
                                         ([("tool", len(prompt) - 1, len(prompt))] if step else [])))
            want = task["start"] + 1 + step
            reward += 0.5 if out["token_ids"] and out["token_ids"][0] == want else 0.0
            prompt = prompt + out["token_ids"] + [3]          # observation token
        return Rollout(env_name=self.name, task_id=task_id, group_id=group_id, turns=turns, reward=reward,
                       policy_version=policy_version, metrics={"reward": reward})


REGISTRY = {"reverse-text": ReverseTextEnv, "copy": CopyEnv, "count-up": CountUpEnv, "low-token": LowTokenEnv}


def load_environment(cfg) -> Environment:
    if cfg.import_path:
        mod, _, attr = cfg.import_path.replace(":", ".").rpartition(".")
        factory = getattr(importlib.import_module(mod), attr)
        env = factory(**cfg.args)
        env.name = cfg.resolved_name
        return env
    if cfg.id == "remote":
        from .env_server import RemoteEnvironment

        return RemoteEnvironment(name=cfg.name, **cfg.args)       # args: base_url = "http://host:port"
    if cfg.id not in REGISTRY:
        raise KeyError(f"unknown environment '{cfg.id}'; built-ins: {sorted(REGISTRY)}")
    return REGISTRY[cfg.id](name=cfg.resolved_name, **cfg.args)
