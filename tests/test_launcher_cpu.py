"""The ``rl`` launcher as real processes on CPU: inference server, orchestrator and trainer started by
``entrypoints/rl.py``, weights broadcast in memory (gloo), eight steps (the orchestrator ships its last batches ahead of the trainer and must
keep answering the trainer's weight offers until the last one), clean exit with nothing left running."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.slow
def test_rl_launcher_runs_three_processes_to_completion(tmp_path, free_ports):
    free_port, broadcast_port = free_ports(2)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "prime_rl_b200.entrypoints.rl", "@", str(ROOT / "examples" / "rl.toml"),
           "--output-dir", str(tmp_path), "--max-steps", "8", "--inference.server.port", str(free_port),
           "--weight-broadcast.type", "nccl", "--weight-broadcast.port", str(broadcast_port)]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    logs = {p.name: p.read_text() for p in tmp_path.rglob("*.log")}
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + "".join(f"\n== {k}\n{v[-1500:]}" for k, v in logs.items())
    assert "trainer and orchestrator finished" in r.stdout
    orch, trainer = logs["orchestrator.log"], logs["trainer.log"]
    assert all(f"step {s} |" in orch for s in range(8))
    import re

    assert max(int(v) for v in re.findall(r"policy v(\d+)", orch)) >= 6            # the weights of step 5 (or later) arrived
    assert all(f"step {s} |" in trainer for s in range(8))


@pytest.mark.slow
def test_rl_launcher_with_a_recurrent_state_family(tmp_path, free_ports):
    """Nemotron-H (Mamba-2 + attention + MoE blocks) through the same three processes: the engine serves it with the
    recurrent-state runner and takes the in-memory weight updates, whose layer groups follow the family's checkpoint
    naming (``backbone.layers``)."""
    cfg = ROOT / "examples" / "rl_hybrid.toml"
    free_port, broadcast_port = free_ports(2)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "prime_rl_b200.entrypoints.rl", "@", str(cfg), "--output-dir", str(tmp_path / "out"),
           "--max-steps", "4", "--inference.server.port", str(free_port),
           "--weight-broadcast.type", "nccl", "--weight-broadcast.port", str(broadcast_port)]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    logs = {p.name: p.read_text() for p in tmp_path.rglob("*.log")}
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:] + "".join(f"\n== {k}\n{v[-1500:]}" for k, v in logs.items())
    import re

    assert max(int(v) for v in re.findall(r"policy v(\d+)", logs["orchestrator.log"])) >= 2
    assert "step 3 |" in logs["trainer.log"]
