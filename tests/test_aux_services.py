"""Env server + remote environment, dashboard API, evals bookkeeping, sbatch rendering (CPU)."""

import json
from pathlib import Path

import httpx
import pytest
from starlette.testclient import TestClient

from prime_rl_b200.configs.orchestrator import EnvConfig


def test_env_server_and_remote_environment():
    from prime_rl_b200.orchestrator.env_server import RemoteEnvironment, build_app
    from prime_rl_b200.orchestrator.envs import load_environment

    env = load_environment(EnvConfig(id="reverse-text"))
    app = build_app(env)
    client = TestClient(app)
    info = client.get("/info").json()
    assert info["name"] == "reverse-text" and info["num_tasks"] == env.num_tasks
    task = client.post("/task", json={"task_id": 3}).json()
    assert task == env.task(3)
    good = task["payload"][::-1]
    assert client.post("/score", json={"task": task, "completion": good}).json()["reward"] == pytest.approx(1.0)
    # the client-side environment talks to the same app through an in-process transport
    class _Bridge(httpx.BaseTransport):
        def handle_request(self, request):
            r = client.request(request.method, request.url.path, content=request.content,
                               headers={"content-type": "application/json"})
            return httpx.Response(r.status_code, content=r.content, headers={"content-type": "application/json"})

    remote = RemoteEnvironment("http://env", transport=_Bridge())
    assert remote.name == "reverse-text" and remote.task(3) == env.task(3)
    assert remote.score(task, good) == pytest.approx(1.0)


def test_dashboard_registry_and_metrics(tmp_path, monkeypatch):
    monkeypatch.setenv("PRL_DASHBOARD_STATE", str(tmp_path / "state"))
    import importlib

    import prime_rl_b200.dashboard.server as srv
    srv = importlib.reload(srv)
    run = tmp_path / "run"
    (run / "logs").mkdir(parents=True)
    (run / "logs" / "metrics.jsonl").write_text(json.dumps({"step": 1, "loss": 0.5}) + "\n" +
                                                json.dumps({"step": 2, "loss": 0.25}) + "\n{\"step\": 3, \"lo")
    srv.register_output_dir(run)
    srv.register_output_dir(run)
    assert srv.registered_dirs() == [str(run.resolve())]
    client = TestClient(srv.build_app())
    assert client.get("/api/runs").json() == [str(run.resolve())]
    rows = client.get("/api/runs/0/metrics").json()
    assert [r["step"] for r in rows] == [1, 2]
    assert client.get("/api/runs/5/metrics").status_code == 404
    assert "<canvas" in client.get("/").text


def test_evals_step_discovery_and_pass_at_k(tmp_path):
    from prime_rl_b200.evals.evals import pass_at_k, published_steps

    for s, done in ((10, True), (20, False), (30, True)):
        d = tmp_path / "broadcasts" / f"step_{s}"
        d.mkdir(parents=True)
        if done:
            (d / ".finished").touch()
    assert published_steps(tmp_path) == [10, 30]
    assert pass_at_k([[0.0, 1.0], [0.0, 0.0], [1.0, 1.0]]) == pytest.approx(2 / 3)


def test_sbatch_rendering_multi_node(tmp_path):
    from prime_rl_b200.configs.rl import RLConfig
    from prime_rl_b200.utils.slurm import render_rl_sbatch

    cfg = RLConfig.model_validate({"deployment": {"type": "multi_node", "num_train_nodes": 2, "num_infer_nodes": 2},
                                   "slurm": {"job_name": "rl-test", "partition": "b200"},
                                   "inference": {}, "output_dir": str(tmp_path)})
    paths = {"trainer": tmp_path / "trainer.json", "orchestrator": tmp_path / "orchestrator.json",
             "inference": tmp_path / "inference.json"}
    text = render_rl_sbatch(cfg, paths)
    assert "#SBATCH --nodes=4" in text and "--job-name=rl-test" in text and "--partition=b200" in text
    assert "--nnodes=2" in text and "prime_rl_b200.trainer.rl.train" in text
    assert "prime_rl_b200.entrypoints.inference" in text and "prime_rl_b200.entrypoints.orchestrator" in text
