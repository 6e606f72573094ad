"""prime_rl_b200: asynchronous RL post-training for one NVSwitch box of B200 GPUs.

Layout
------
configs/       pydantic config trees and the ``@ file.toml`` + dotted-flag command line
entrypoints/   ``rl``, ``sft``, ``trainer``, ``orchestrator``, ``inference``, ``evals``, ``env-server``
csrc/, native/ hand-written sm_100a CUDA kernels (tcgen05 / TMEM / TMA) and the C++ CPU optimizer
ops/           Python front ends of the kernels with fp32 PyTorch reference implementations
models/        layers and model families (dense, MoE), HF <-> native checkpoint conversion
parallel/      process-group world, parallel dims / meshes, sharded parameters, EP, CP, symmetric memory
trainer/       RL and SFT loops, losses, data, packing, optimizers, checkpoints
engine/        rollout engine: paged KV cache, scheduler, sampler, HTTP server
orchestrator/  asynchronous rollout scheduling, advantages, batching, weight-version tracking
transports/    micro-batch and weight transports between the processes
monitors/      metrics sinks;  utils/  logging, paths, process supervision
"""

__version__ = "0.1.0"
