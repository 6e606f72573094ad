"""Rollout records that flow from the environments through the sinks to the packer."""

from __future__ import annotations

import uuid
from dataclasses import dataclass, field
from typing import Any


@dataclass
class Turn:
    """One model call inside an episode: the context it saw and what it sampled."""

    prompt_ids: list[int]
    completion_ids: list[int]
    completion_logprobs: list[float]
    temperature: float = 1.0
    routed_experts: Any | None = None      # np.ndarray [tokens, layers, k] for the completion
    sampling_mask: Any | None = None       # (ids int32, counts int32) for the completion
    finish_reason: str | None = None
    role_spans: list[tuple[str, int, int]] = field(default_factory=list)   # (role, start, end) over prompt tokens
    # image inputs of the prompt: {"pixel_values": float array [patches, patch_dim], "image_grid_thw": [[t, h, w], ...],
    # "image_token_id": id of the placeholder tokens in prompt_ids}; they go to the engine with the request and to the
    # trainer with the sample
    mm: dict | None = None


@dataclass
class Rollout:
    """One episode of one task: a linear chain of turns where every turn's prompt extends the
    previous turn's prompt + completion (multi-turn environments append observation tokens)."""

    env_name: str
    task_id: int
    group_id: str
    turns: list[Turn]
    reward: float = 0.0
    policy_version: int = 0
    metrics: dict[str, float] = field(default_factory=dict)
    info: dict[str, Any] = field(default_factory=dict)
    trace_id: str = field(default_factory=lambda: uuid.uuid4().hex)
    agent: str | None = None
    error: str | None = None
    # filled by the algorithm
    advantage: float | None = None

    @property
    def num_output_tokens(self) -> int:
        return sum(len(t.completion_ids) for t in self.turns)

    @property
    def num_total_tokens(self) -> int:
        last = self.turns[-1]
        return len(last.prompt_ids) + len(last.completion_ids)

    @property
    def num_turns(self) -> int:
        return len(self.turns)


@dataclass
class Policy:
    version: int = 0
