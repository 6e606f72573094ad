"""Distributed runtime: world, parallel dims, sharded parameters, expert / context parallelism."""

from .dims import ParallelDims, get_parallel_dims, resolve_ep  # noqa: F401
from .world import World, get_world, reset_world, setup_distributed  # noqa: F401
