"""``inference @ inference.toml``: builds the model, the engine and serves the HTTP API
(reference: src/prime_rl/entrypoints/inference.py:192-253)."""

from __future__ import annotations

from pathlib import Path

import torch

from ..configs.base import cli
from ..configs.inference import InferenceConfig
from ..utils.logger import setup_logger


def build_engine(config: InferenceConfig, tp=None):
    """``tp``: the ``engine/tp.py`` context of a tensor-parallel launch (this process holds one shard)."""
    from ..engine.engine import Engine
    from ..models import build_model, resolve_arch
    from ..trainer.weights import load_hf_checkpoint

    ec = config.vllm
    arch = resolve_arch(ec.model, ec.arch)
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    if tp is not None:
        device = tp.device
    dtype = {"auto": torch.bfloat16 if device.type == "cuda" else torch.float32, "bfloat16": torch.bfloat16,
             "float16": torch.float16, "float32": torch.float32}[ec.dtype]
    model = build_model(arch, device=device, dtype=dtype, seed=ec.seed)
    if tp is not None and tp.size > 1:
        from ..engine.tp import shard_model_

        # before the checkpoint load: every rank reads only its slices
        shard_model_(model, tp.rank, tp.size, expert_parallel=bool(ec.enable_expert_parallel) and arch.is_moe)
    if Path(ec.model).is_dir() and not ec.random_init:
        load_hf_checkpoint(model, Path(ec.model), strict=False)
    for p in model.parameters():
        p.requires_grad_(False)
    if ec.num_pages is not None:
        pages = ec.num_pages
    elif device.type == "cuda":
        free, total = torch.cuda.mem_get_info(device)
        per_page = 2 * arch.num_hidden_layers * ec.page_size * arch.kv_dim * torch.empty((), dtype=dtype).element_size()
        per_page //= tp.size if tp is not None else 1
        pages = max(64, int((free - (1.0 - ec.gpu_memory_utilization) * total) // per_page))
    else:
        pages = 2048
    vision_kw = {}
    if ec.vlm is not None:
        from ..models.vision import VisionConfig, VisionTower

        vc = VisionConfig(**{"out_hidden_size": arch.hidden_size, **ec.vlm.vision})
        tower = VisionTower(vc, dtype=dtype, device=device).eval()
        for p in tower.parameters():
            p.requires_grad_(False)
        if Path(ec.model).is_dir() and not ec.random_init:
            from ..trainer.weights import load_vision_tower

            load_vision_tower(tower, Path(ec.model))
        vision_kw = dict(vision=tower, image_token_id=ec.vlm.image_token_id, mrope_section=tuple(ec.vlm.mrope_section))
    engine = Engine(model, num_pages=pages, page_size=ec.page_size, max_running=ec.max_num_seqs, **vision_kw,
                    max_prefill_tokens=ec.max_num_batched_tokens,
                    enable_prefix_cache=ec.enable_prefix_caching is not False, tp=tp,
                    kv_offload_bytes=_kv_offload_bytes(config),
                    expert_parallel=bool(ec.enable_expert_parallel) and arch.is_moe)
    engine.runner.capture_routed = ec.enable_return_routed_experts and arch.is_moe
    return engine


def _kv_offload_bytes(config: InferenceConfig) -> int:
    """Host-memory budget for the K / V of preempted requests (``kv_cache_offload.cpu.num_bytes``)."""
    off = config.kv_cache_offload
    return int(off.cpu.num_bytes) if off is not None and off.cpu is not None else 0


def load_tokenizer(name: str):
    try:
        if Path(name).is_dir():
            from transformers import AutoTokenizer

            return AutoTokenizer.from_pretrained(name)
    except Exception:
        pass
    return None


def serve(config: InferenceConfig) -> None:
    import uvicorn

    from ..engine.server import build_app

    _serve_engine(build_engine(config).start(), config)


def _serve_engine(engine, config: InferenceConfig) -> None:
    import uvicorn

    from ..engine.server import build_app

    app = build_app(engine, config.vllm.model, tokenizer=load_tokenizer(config.vllm.model),
                    liveness_timeout=config.server.liveness_timeout_seconds)
    app.state.return_sampling_mask = config.enable_return_sampling_mask
    uvicorn.run(app, host=config.server.host or "0.0.0.0", port=config.server.port, log_level="warning")


def serve_tensor_parallel(config: InferenceConfig, argv: list[str]) -> int:
    """``tensor_parallel_size`` processes, one GPU each. Outside a ``torchrun`` environment this
    relaunches the same command line under it; inside, rank 0 serves HTTP and drives the step loop,
    the other ranks follow its announcements (``Engine.follow``)."""
    import os
    import subprocess
    import sys

    n = config.vllm.tensor_parallel_size
    if "LOCAL_RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
               "127.0.0.1", "--master-port", str(config.vllm.data_parallel_rpc_port), "-m",
               "prime_rl_b200.entrypoints.inference", *argv]
        return subprocess.call(cmd)
    from ..engine.tp import init_tp
    from ..models import resolve_arch

    arch = resolve_arch(config.vllm.model, config.vllm.arch)
    if int(os.environ.get("WORLD_SIZE", "1")) != n:
        raise ValueError(f"tensor_parallel_size={n} but the launch has {os.environ.get('WORLD_SIZE')} processes")
    tp = init_tp(max(config.vllm.max_num_batched_tokens, 8192), arch.hidden_size)
    engine = build_engine(config, tp=tp)
    if tp.rank == 0:
        _serve_engine(engine.start(), config)
        engine.shutdown()
    else:
        engine.follow()
    return 0


def serve_replicas(config: InferenceConfig, argv: list[str], prefill_replicas: int = 0) -> int:
    """Data-parallel serving on one node: ``data_parallel_size`` engine processes, one GPU each, on
    the ports after ``server.port``, and the request router (``engine/router.py``) on ``server.port``
    in this process. The children get the same command line plus their own port and a replica
    count of one; the first child that dies takes the service down.

    ``prefill_replicas`` > 0 (``deployment.type = "disaggregated"`` on one node): that many more engine
    processes that only run prompts; the router sends every request to one of them first and hands its K / V
    (a file in shared memory) and first token to one of the ``data_parallel_size`` decode engines."""
    import os
    import subprocess
    import sys
    import time

    import httpx
    import uvicorn

    from ..engine.router import Router, build_app
    from ..utils.process import Supervisor

    decode_n, port = config.vllm.data_parallel_size, config.server.port
    n = decode_n + prefill_replicas
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    gpus = [g for g in visible.split(",") if g] if visible is not None else [str(i) for i in range(n)]
    tp = config.vllm.tensor_parallel_size                # every replica may itself span several GPUs
    if prefill_replicas and tp > 1:
        raise ValueError("prefill / decode disaggregation runs single-GPU engines (the K / V hand-off is per process)")
    if visible != "" and len(gpus) < n * tp:
        raise ValueError(f"{n} replicas x tensor_parallel_size={tp} but only {len(gpus)} GPUs are visible")
    sup = Supervisor()
    urls = []
    for i in range(n):
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(gpus[i * tp:(i + 1) * tp]))
        env["PRIME_RL_ENGINE_CHILD"] = "1"             # the child serves one engine whatever the deployment says
        cmd = [sys.executable, "-m", "prime_rl_b200.entrypoints.inference", *argv, "--vllm.data-parallel-size", "1",
               "--server.port", str(port + 1 + i), "--server.host", "127.0.0.1", "--vllm.data-parallel-rpc-port",
               str(config.vllm.data_parallel_rpc_port + i)]
        sup.add(f"replica{i}", subprocess.Popen(cmd, env=env))
        urls.append(f"http://127.0.0.1:{port + 1 + i}")
    deadline = time.time() + 1800
    for u in urls:                                  # the router answers /health only once every replica does
        while True:
            try:
                if httpx.get(u + "/health", timeout=5).status_code == 200:
                    break
            except httpx.HTTPError:
                pass
            if not sup.errors.empty() or time.time() > deadline:
                sup.shutdown()
                raise RuntimeError("an engine replica did not come up")
            time.sleep(1.0)
    router = Router(urls[:decode_n], prefill_urls=urls[decode_n:])      # the first ``decode_n`` processes decode
    server = uvicorn.Server(uvicorn.Config(build_app(router), host=config.server.host or "0.0.0.0", port=port,
                                           log_level="warning"))
    import threading

    def watch():
        sup.errors.get()                            # blocks until a replica exits with an error
        server.should_exit = True

    threading.Thread(target=watch, daemon=True).start()
    try:
        server.run()
    finally:
        sup.shutdown()
    return 0


def main(argv: list[str] | None = None) -> None:
    import sys

    args = list(sys.argv[1:] if argv is None else argv)
    config = cli(InferenceConfig, args)
    if config.dry_run:
        print(config.to_json())
        return
    setup_logger(config.log.level, tag="inference", json_logging=config.log.json_logging)
    import os

    dep = config.deployment
    if dep.type == "disaggregated" and config.slurm is None and not os.environ.get("PRIME_RL_ENGINE_CHILD"):
        # one node: ``num_decode_replicas`` decode engines and ``num_prefill_replicas`` prefill engines behind the router
        config.vllm.data_parallel_size = dep.num_decode_replicas
        serve_replicas(config, args, prefill_replicas=dep.num_prefill_replicas)
        return
    if config.vllm.data_parallel_size > 1:
        serve_replicas(config, args)
        return
    if config.vllm.tensor_parallel_size > 1:
        serve_tensor_parallel(config, args)
        return
    serve(config)


if __name__ == "__main__":
    main()
