"""End-to-end asynchronous RL on CPU in one process: rollout engine behind its HTTP app,
orchestrator (dispatcher, GRPO, packing, watcher) and trainer, connected by the filesystem
batch transport and the filesystem weight broadcast."""

import asyncio
import json
import threading

import httpx
import pytest
import torch

from prime_rl_b200.configs.orchestrator import OrchestratorConfig
from prime_rl_b200.configs.trainer import TrainerConfig
from prime_rl_b200.engine.engine import Engine
from prime_rl_b200.engine.server import build_app
from prime_rl_b200.models import build_model, resolve_arch
from prime_rl_b200.orchestrator.orchestrator import Orchestrator
from prime_rl_b200.trainer.rl.train import RLTrainer
from prime_rl_b200.utils.logger import setup_logger


@pytest.mark.slow
def test_async_rl_three_steps(tmp_path):
    setup_logger("warning")
    run_dir = tmp_path / "run"
    arch = resolve_arch("tiny-qwen3")
    engine = Engine(build_model(arch, device="cpu", dtype=torch.float32), num_pages=512).start()
    app = build_app(engine, "tiny-qwen3")
    steps = 3

    tcfg = TrainerConfig.model_validate({
        "model": {"name": "tiny-qwen3", "seq_len": 128, "ac": None, "debug": {"random_init": True}},
        "optim": {"lr": 1e-3}, "max_steps": steps, "output_dir": str(run_dir),
        "rollout_transport": {"type": "filesystem"}, "weight_broadcast": {"type": "filesystem"}})
    ocfg = OrchestratorConfig.model_validate({
        "model": {"name": "tiny-qwen3", "client": {"base_url": "http://engine/v1", "wait_for_ready_timeout": 30}},
        "train": {"source": [{"id": "reverse-text", "args": {"vocab_size": arch.vocab_size, "max_len": 6}}],
                  "sampling": {"temperature": 1.0, "max_completion_tokens": 6}},
        "batch_size": 8, "group_size": 4, "seq_len": 128, "max_steps": steps, "output_dir": str(run_dir),
        "rollout_transport": {"type": "filesystem"}, "weight_broadcast": {"type": "filesystem"},
        "concurrency": {"initial_inflight": 8, "max_inflight": 16}, "collect_inference_metrics": False})

    errors = []

    def trainer_thread():
        try:
            RLTrainer(tcfg, device=torch.device("cpu")).setup().run()
        except Exception as e:  # surfaced in the main thread below
            errors.append(e)

    th = threading.Thread(target=trainer_thread, daemon=True)
    th.start()

    async def go():
        orch = await Orchestrator(ocfg, http_transport=httpx.ASGITransport(app=app)).setup()
        await asyncio.wait_for(orch.run(), timeout=300)
        return orch

    orch = asyncio.run(go())
    th.join(timeout=120)
    engine.shutdown()
    assert not errors, errors
    assert not th.is_alive()
    assert orch.step == steps
    # the engine took at least the first policy update while the run was going
    assert engine.policy_version >= 1 and orch.policy.version >= 1
    rows = [json.loads(l) for l in (run_dir / "monitors" / "file" / "metrics.jsonl").read_text().splitlines()]
    producers = {r["producer"] for r in rows}
    assert producers == {"trainer", "orchestrator"}
    tr = [r for r in rows if r["producer"] == "trainer"]
    assert len(tr) == steps and all(r["loss"] == r["loss"] for r in tr)
    assert (run_dir / "broadcasts").exists() and (run_dir / "batches" / "step_0" / "rank_0.bin").exists()
