"""Failure detection exercised on the host only: a child that dies, a rank that never joins,
an engine that answers 5xx, a handshake nobody acknowledges, a truncated checkpoint."""

import os
import subprocess
import sys
import textwrap
import time

import httpx
import pytest
import torch

from prime_rl_b200.utils.process import Supervisor, popen


def test_supervisor_reports_first_failure_and_kills_the_rest(tmp_path):
    sup = Supervisor()
    env = dict(os.environ)
    sup.add("long", popen([sys.executable, "-c", "import time; time.sleep(60)"], env, tmp_path / "long.log"))
    sup.add("bad", popen([sys.executable, "-c", "import sys; sys.exit(7)"], env, tmp_path / "bad.log"))
    t0 = time.monotonic()
    failure = sup.wait(required=["long", "bad"])
    assert failure == ("bad", 7)
    sup.shutdown()
    assert sup.children["long"].poll() is not None and time.monotonic() - t0 < 30


def test_rank_that_never_joins_ends_the_collective_with_an_error(tmp_path, free_port):
    """Two gloo ranks; rank 1 exits before the all-reduce. Rank 0's collective fails within the
    process-group timeout instead of hanging."""
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import datetime, os, sys, torch, torch.distributed as dist
        rank = int(sys.argv[1])
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{free_port}", rank=rank, world_size=2,
                                timeout=datetime.timedelta(seconds=5))
        dist.barrier()
        if rank == 1:
            os._exit(3)                      # leaves between steps, nothing in flight
        try:
            dist.all_reduce(torch.ones(4))
        except Exception as e:
            print("DETECTED", type(e).__name__)
            sys.exit(0)
        sys.exit(9)
    """))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, text=True) for r in range(2)]
    out0, _ = procs[0].communicate(timeout=120)
    procs[1].wait(timeout=120)
    assert procs[1].returncode == 3
    assert procs[0].returncode == 0 and "DETECTED" in out0


def test_inference_client_retries_5xx_then_raises():
    from prime_rl_b200.configs.shared import ClientConfig
    from prime_rl_b200.orchestrator.clients import InferenceClient

    calls = {"n": 0}

    def handler(request):
        calls["n"] += 1
        return httpx.Response(503, json={"error": "overloaded"})

    import asyncio

    async def run():
        c = InferenceClient(ClientConfig(), "m", retries=3, transport=httpx.MockTransport(handler))
        sampling = type("S", (), {"temperature": 1.0, "top_p": 1.0, "max_completion_tokens": 4, "extra_body": {}})()
        with pytest.raises(httpx.HTTPStatusError):
            await c.generate([1, 2, 3], sampling)
        await c.close()

    asyncio.run(run())
    assert calls["n"] == 3


def test_weight_handshake_without_receiver_times_out(tmp_path):
    from prime_rl_b200.parallel.world import World
    from prime_rl_b200.transports.weights import SENDER_READY, WeightSender

    class Sender(WeightSender):
        def _broadcast(self, model, step, d):
            raise AssertionError("must not transfer without an acknowledgement")

    cfg = type("C", (), {"timeout": 0.3, "type": "nccl"})()
    s = Sender(cfg, tmp_path, World(), require_ack=True)
    with pytest.raises(TimeoutError):
        s.broadcast(None, 4)
    assert (s.step_dir(4) / SENDER_READY).exists()


def test_truncated_checkpoint_is_an_error_not_a_silent_partial_load(tmp_path):
    from prime_rl_b200.models import build_model, resolve_arch
    from prime_rl_b200.trainer.ckpt import CheckpointManager, Progress

    model = build_model(resolve_arch("tiny-qwen3"), device="cpu", dtype=torch.float32, seed=0)
    mgr = CheckpointManager(tmp_path, None)
    path = mgr.save(1, model, None, Progress())
    shard = max(path.glob("*.distcp"), key=lambda f: f.stat().st_size)
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 3])
    with pytest.raises(Exception):
        mgr.load(1, build_model(resolve_arch("tiny-qwen3"), device="cpu", dtype=torch.float32, seed=1), None, Progress())
