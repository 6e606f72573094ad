"""Parallel dimensions and the process groups derived from them.

Rank layout (outer to inner): ``dp_replicate x dp_shard x cp``; expert parallelism reuses
the ``dp_shard x cp`` ranks (``ep`` consecutive ranks form one EP group), as in the
reference (src/prime_rl/trainer/parallel_dims.py:36-153, :287-315). Pipeline parallelism is
fixed to 1 there and here.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch.distributed as dist


@dataclass
class ParallelDims:
    world_size: int
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    ep: int = 1
    pp: int = 1
    _groups: dict = field(default_factory=dict, repr=False)

    def __post_init__(self):
        if self.dp_shard == -1:
            denom = self.dp_replicate * self.cp * self.pp
            if self.world_size % denom:
                raise ValueError(f"world_size {self.world_size} not divisible by dp_replicate*cp*pp = {denom}")
            self.dp_shard = self.world_size // denom
        if self.dp_replicate * self.dp_shard * self.cp * self.pp != self.world_size:
            raise ValueError("dp_replicate * dp_shard * cp * pp must equal world_size")
        if self.pp != 1:
            raise ValueError("pipeline parallelism is not supported (pp must be 1)")
        if self.ep > 1:
            if self.ep % self.cp:
                raise ValueError("ep must be a multiple of cp")
            if (self.dp_shard * self.cp) % self.ep:
                raise ValueError("dp_shard * cp must be a multiple of ep")

    # ------------------------------------------------------------------ sizes
    @property
    def dp(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def dp_shard_cp(self) -> int:
        return self.dp_shard * self.cp

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def ep_enabled(self) -> bool:
        return self.ep > 1

    @property
    def fsdp_gradient_divide_factor(self) -> int:
        """Gradients are summed over every dp x cp rank (losses are pre-divided by global
        token counts), so the data-parallel mean must be undone by this factor."""
        return self.dp_replicate * self.dp_shard * self.cp

    # ------------------------------------------------------------------ coordinates
    def coords(self, rank: int) -> dict[str, int]:
        cp_rank = rank % self.cp
        shard_rank = (rank // self.cp) % self.dp_shard
        rep_rank = rank // (self.cp * self.dp_shard)
        inner = rank % self.dp_shard_cp
        return dict(cp=cp_rank, dp_shard=shard_rank, dp_replicate=rep_rank, dp=rep_rank * self.dp_shard + shard_rank,
                    dp_shard_cp=inner, ep=inner % self.ep if self.ep > 1 else 0,
                    dp_shard_mod_ep=inner // self.ep if self.ep > 1 else inner)

    def _rank_lists(self, name: str) -> list[list[int]]:
        W, cp, ds, dr, ep = self.world_size, self.cp, self.dp_shard, self.dp_replicate, self.ep
        inner = cp * ds
        if name == "cp":
            return [list(range(s, s + cp)) for s in range(0, W, cp)]
        if name == "dp_shard_cp":
            return [list(range(s, s + inner)) for s in range(0, W, inner)]
        if name == "dp_replicate":
            return [[r * inner + i for r in range(dr)] for i in range(inner)]
        if name == "dp_cp" or name == "world":
            return [list(range(W))]
        if name == "dp":
            return [[d * cp + c for d in range(dr * ds)] for c in range(cp)]
        if name == "dp_shard":
            return [[r * inner + s * cp + c for s in range(ds)] for r in range(dr) for c in range(cp)]
        if name == "ep":
            return [list(range(s, s + ep)) for s in range(0, W, ep)] if ep > 1 else [[r] for r in range(W)]
        if name == "ep_replicas":  # ranks that hold the same expert shard
            if ep <= 1:
                return [list(range(W))]
            return [[i + j * ep for j in range(W // ep)] for i in range(ep)]
        if name == "dp_shard_mod_ep":
            if ep <= 1:
                return self._rank_lists("dp_shard_cp")
            return [[r * inner + j * ep + i for j in range(inner // ep)] for r in range(dr) for i in range(ep)]
        raise KeyError(name)

    def group_ranks(self, name: str, rank: int) -> list[int]:
        for ranks in self._rank_lists(name):
            if rank in ranks:
                return ranks
        raise ValueError(f"rank {rank} not in any '{name}' group")

    def group(self, name: str):
        """Process group of this rank for mesh dimension ``name`` (None when single-process
        or the group is the whole world, which maps to the default group)."""
        if not dist.is_initialized():
            return None
        if name in self._groups:
            return self._groups[name]
        lists = self._rank_lists(name)
        mine = None
        me = dist.get_rank()
        if len(lists) == 1 and len(lists[0]) == self.world_size:
            mine = dist.group.WORLD
        else:
            for ranks in lists:  # every rank must create every group, in the same order
                g = dist.new_group(ranks=ranks)
                if me in ranks:
                    mine = g
        self._groups[name] = mine
        return mine

    def group_size(self, name: str) -> int:
        return len(self._rank_lists(name)[0])

    def local_rank(self, name: str, rank: int | None = None) -> int:
        rank = dist.get_rank() if rank is None and dist.is_initialized() else (rank or 0)
        return self.group_ranks(name, rank).index(rank)


def resolve_ep(ep: int | str, *, is_moe: bool, world_size: int, dp_replicate: int = 1, num_experts: int = 0) -> int:
    """``ep="auto"`` -> min(world / dp_replicate, 8) for MoE models (largest divisor of the
    expert count that fits), 1 for dense models."""
    if ep != "auto":
        return int(ep)
    if not is_moe:
        return 1
    cand = min(world_size // dp_replicate, 8)
    while cand > 1 and (num_experts % cand or (world_size // dp_replicate) % cand):
        cand -= 1
    return max(cand, 1)


def get_parallel_dims(model_cfg, world_size: int, *, is_moe: bool = False, num_experts: int = 0) -> ParallelDims:
    ep = resolve_ep(model_cfg.ep, is_moe=is_moe, world_size=world_size, dp_replicate=model_cfg.dp_replicate,
                    num_experts=num_experts)
    return ParallelDims(world_size=world_size, dp_replicate=model_cfg.dp_replicate, cp=model_cfg.cp, ep=ep)
