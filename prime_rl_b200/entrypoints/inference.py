"""``inference @ inference.toml``: builds the model, the engine and serves the HTTP API
(reference: src/prime_rl/entrypoints/inference.py:192-253)."""

from __future__ import annotations

from pathlib import Path

import torch

from ..configs.base import cli
from ..configs.inference import InferenceConfig
from ..utils.logger import setup_logger


def build_engine(config: InferenceConfig):
    from ..engine.engine import Engine
    from ..models import build_model, resolve_arch
    from ..trainer.weights import load_hf_checkpoint

    ec = config.vllm
    arch = resolve_arch(ec.model, ec.arch)
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    dtype = {"auto": torch.bfloat16 if device.type == "cuda" else torch.float32, "bfloat16": torch.bfloat16,
             "float16": torch.float16, "float32": torch.float32}[ec.dtype]
    model = build_model(arch, device=device, dtype=dtype, seed=ec.seed)
    if Path(ec.model).is_dir() and not ec.random_init:
        load_hf_checkpoint(model, Path(ec.model), strict=False)
    for p in model.parameters():
        p.requires_grad_(False)
    if ec.num_pages is not None:
        pages = ec.num_pages
    elif device.type == "cuda":
        free, total = torch.cuda.mem_get_info(device)
        per_page = 2 * arch.num_hidden_layers * ec.page_size * arch.kv_dim * torch.empty((), dtype=dtype).element_size()
        pages = max(64, int((free - (1.0 - ec.gpu_memory_utilization) * total) // per_page))
    else:
        pages = 2048
    engine = Engine(model, num_pages=pages, page_size=ec.page_size, max_running=ec.max_num_seqs,
                    max_prefill_tokens=ec.max_num_batched_tokens,
                    enable_prefix_cache=ec.enable_prefix_caching is not False)
    engine.runner.capture_routed = ec.enable_return_routed_experts and arch.is_moe
    return engine


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

    engine = build_engine(config).start()
    app = build_app(engine, config.vllm.model, tokenizer=load_tokenizer(config.vllm.model),
                    liveness_timeout=config.server.liveness_timeout_seconds)
    app.state.return_sampling_mask = config.enable_return_sampling_mask
    uvicorn.run(app, host=config.server.host or "0.0.0.0", port=config.server.port, log_level="warning")


def main(argv: list[str] | None = None) -> None:
    config = cli(InferenceConfig, argv)
    if config.dry_run:
        print(config.to_json())
        return
    setup_logger(config.log.level, tag="inference", json_logging=config.log.json_logging)
    serve(config)


if __name__ == "__main__":
    main()
