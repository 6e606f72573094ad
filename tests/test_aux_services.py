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


def _bash_syntax_ok(text: str, tmp_path, name: str) -> None:
    import subprocess

    p = tmp_path / name
    p.write_text(text)
    r = subprocess.run(["bash", "-n", str(p)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_sbatch_rendering_multi_node(tmp_path):
    from prime_rl_b200.configs.rl import RLConfig
    from prime_rl_b200.utils.slurm import render_rl_sbatch

    cfg = RLConfig.model_validate({"deployment": {"type": "multi_node", "num_train_nodes": 2, "num_infer_nodes": 2},
                                   "slurm": {"job_name": "rl-test", "partition": "b200", "account": "acct",
                                             "cleanup_grace_period": 120, "pre_run_command": "module load cuda"},
                                   "env_vars": {"NCCL_DEBUG": "WARN", "ODD": "a b"},
                                   "inference": {}, "output_dir": str(tmp_path)})
    paths = {"trainer": tmp_path / "trainer.json", "orchestrator": tmp_path / "orchestrator.json",
             "inference": tmp_path / "inference.json"}
    text = render_rl_sbatch(cfg, paths)
    _bash_syntax_ok(text, tmp_path, "rl.sbatch")
    assert "#SBATCH --nodes=4" in text and "--job-name=rl-test" in text and "--partition=b200" in text
    assert "#SBATCH --account=acct" in text and "#SBATCH --time" not in text
    assert "NUM_TRAIN_NODES=2" in text and "NUM_INFER_NODES=2" in text and "prime_rl_b200.trainer.rl.train" in text
    assert "prime_rl_b200.entrypoints.inference" in text and "prime_rl_b200.entrypoints.orchestrator" in text
    assert "prime_rl_b200.engine.router" in text and "--kill-on-bad-exit=1" in text
    assert "export ODD='a b'" in text and "module load cuda" in text and "holding for 120s" in text
    assert "ORCH_PROCID=$NUM_INFER_NODES" in text           # beside trainer rank 0 by default
    assert "pkill" not in text and "killall" not in text    # leftovers are ended by recorded pid only
    cfg2 = RLConfig.model_validate({"deployment": {"type": "multi_node", "num_train_nodes": 1, "num_infer_nodes": 2,
                                                   "orchestrator_on_inference": True},
                                    "inference": {}, "output_dir": str(tmp_path)})
    text2 = render_rl_sbatch(cfg2, paths)
    _bash_syntax_ok(text2, tmp_path, "rl2.sbatch")
    assert "ORCH_PROCID=$((NUM_INFER_NODES - 1))" in text2


def test_sbatch_rendering_other_launchers_and_user_templates(tmp_path):
    from types import SimpleNamespace

    from prime_rl_b200.configs.inference import InferenceConfig
    from prime_rl_b200.configs.rl import RLConfig
    from prime_rl_b200.configs.shared import SlurmConfig
    from prime_rl_b200.utils.slurm import render_inference_sbatch, render_rl_sbatch, render_sft_sbatch

    view = SimpleNamespace(slurm=SlurmConfig(job_name="sft"), run_dir=tmp_path, env_vars={})
    one = render_sft_sbatch(view, tmp_path / "sft.json", nodes=1, gpus_per_node=4)
    many = render_sft_sbatch(view, tmp_path / "sft.json", nodes=3, gpus_per_node=8)
    _bash_syntax_ok(one, tmp_path, "sft1.sbatch")
    _bash_syntax_ok(many, tmp_path, "sft3.sbatch")
    assert "--nproc-per-node=4" in one and "#SBATCH --nodes=1" in one and "--master-addr=127.0.0.1" in one
    assert "#SBATCH --nodes=3" in many and "--node-rank=$SLURM_PROCID" in many and "NUM_NODES=3" in many

    inf = InferenceConfig.model_validate({"deployment": {"type": "disaggregated", "prefill_nodes_per_replica": 1,
                                                         "decode_nodes_per_replica": 2,
                                                         "prefill_env_vars": {"ROLE_HINT": "p"}},
                                          "vllm": {"tensor_parallel_size": 2}, "slurm": {"job_name": "inf"}})
    inf_view = SimpleNamespace(slurm=inf.slurm, run_dir=tmp_path, env_vars={}, vllm=inf.vllm, server=inf.server,
                               deployment=inf.deployment)
    text = render_inference_sbatch(inf_view, tmp_path / "inference.json", nodes=3, gpus_per_node=8)
    _bash_syntax_ok(text, tmp_path, "inf.sbatch")
    assert "PRL_INFERENCE_ROLE=prefill" in text and "--vllm.tensor-parallel-size 2" in text
    assert "--vllm.data-parallel-size 4" in text and "prime_rl_b200.engine.router" in text

    # single-node RL under SLURM hands over to the local launcher
    cfg = RLConfig.model_validate({"slurm": {"job_name": "one"}, "inference": {}, "output_dir": str(tmp_path)})
    single = render_rl_sbatch(cfg, {"rl": tmp_path / "rl.json", "trainer": tmp_path / "trainer.json",
                                    "orchestrator": tmp_path / "orchestrator.json"})
    _bash_syntax_ok(single, tmp_path, "one.sbatch")
    assert "prime_rl_b200.entrypoints.rl @" in single and "--slurm None" in single

    # a user template sees the same variables and may include the stock pieces
    user = tmp_path / "mine.j2"
    user.write_text('{% include "_header.sbatch.j2" %}\necho train={{ num_train_nodes }} infer={{ num_infer_nodes }} '
                    'tp={{ inference_tp }} cfg={{ config_dir }}\n')
    cfg3 = RLConfig.model_validate({"deployment": {"type": "multi_node", "num_train_nodes": 2, "num_infer_nodes": 1},
                                    "slurm": {"template_path": str(user)}, "inference": {},
                                    "output_dir": str(tmp_path)})
    mine = render_rl_sbatch(cfg3, {"trainer": tmp_path / "c" / "trainer.json",
                                   "orchestrator": tmp_path / "c" / "orchestrator.json"})
    assert "echo train=2 infer=1 tp=1" in mine and f"cfg={tmp_path / 'c'}" in mine and "#SBATCH --nodes=3" in mine


def test_trainer_annotations_reach_the_file_monitor(tmp_path):
    import json
    from types import SimpleNamespace

    import torch

    from prime_rl_b200.monitors import FileMonitor, MultiMonitor
    from prime_rl_b200.trainer.rl.annotations import AnnotationWriter

    mon = MultiMonitor([FileMonitor(tmp_path, "trainer")])
    w = AnnotationWriter(mon)
    mb = SimpleNamespace(sequence_lengths=[3, 2, 4], trace_ids=["a", "", "b"], branch_indices=[0, -1, 2],
                         loss_mask=torch.tensor([0, 1, 1, 0, 0, 0, 1, 1, 1], dtype=torch.bool))
    w.collect(mb, torch.arange(9).float() * -0.5, torch.ones(9), step=7)
    assert w.flush() == 2
    files = list(tmp_path.rglob("annotations_trainer.jsonl"))
    rows = [json.loads(l) for l in files[0].read_text().splitlines()]
    assert [r["trace_id"] for r in rows] == ["a", "b"] and rows[1]["branch_index"] == 2 and rows[0]["step"] == 7
    assert rows[1]["logprobs"] == [-2.5, -3.0, -3.5, -4.0] and rows[0]["loss_mask"] == [False, True, True]
    assert w.flush() == 0


def test_chat_session_keeps_history_and_handles_commands():
    import httpx

    from prime_rl_b200.engine.chat import ChatSession

    seen = []

    def handler(request: httpx.Request) -> httpx.Response:
        import json as _json

        if request.url.path == "/v1/models":
            return httpx.Response(200, json={"data": [{"id": "m"}]})
        body = _json.loads(request.content)
        seen.append(body)
        return httpx.Response(200, json={"choices": [{"message": {"role": "assistant",
                                                                  "content": f"reply {len(body['messages'])}"}}]})

    chat = ChatSession("http://x", system="be brief", transport=httpx.MockTransport(handler))
    assert chat.say("hi") == "reply 2"
    assert chat.say("again") == "reply 4"
    assert seen[1]["messages"][0] == {"role": "system", "content": "be brief"} and seen[1]["model"] == "m"
    assert chat.command("/temp 0.2") == "temperature 0.2" and chat.command("hello") is None
    assert chat.command("/reset") == "conversation cleared" and chat.messages == []


def test_benchmark_runner_config_and_result_table(tmp_path):
    import importlib.util
    import json

    def load(name):
        path = Path(__file__).resolve().parents[1] / "benchmarks" / f"{name}.py"
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    run, agg = load("run_single_benchmark"), load("aggregate_results")
    cfg = run.build_config(run.parse_args(["--model-name", "qwen3-30b-a3b", "--lora-rank", "16", "--num-gpus", "8",
                                           "--ac", "Offload", "--output", str(tmp_path / "r.json")]))
    assert cfg["model"]["lora"] == {"rank": 16, "alpha": 32.0} and cfg["data"]["fake"]["batch_size"] == 16
    assert cfg["model"]["ac_offloading"] == {"pin_memory": True}
    from prime_rl_b200.configs.trainer import TrainerConfig

    TrainerConfig.model_validate(cfg)
    good = {"config": {"type": "rl", "model_name": "m", "num_gpus": 8, "success": True, "seq_len": 16384, "lora_rank": 16},
            "metrics": {"throughput": {"mean": 9266.0}, "mfu": {"mean": 7.8}, "step_time": {"mean": 28.3},
                        "peak_memory": {"gib": 100.0}}}
    bad = {"config": {"success": False}, "metrics": {}}
    (tmp_path / "a.json").write_text(json.dumps(good))
    (tmp_path / "b.json").write_text(json.dumps(bad))
    assert agg.main([str(tmp_path / "a.json"), str(tmp_path / "b.json"), "--output", str(tmp_path / "t.md")]) == 0
    text = (tmp_path / "t.md").read_text()
    assert "9266.00" in text and text.count("\n") == 3


def test_dashboard_trace_browser_joins_traces_and_annotations(tmp_path, monkeypatch):
    from fastapi.testclient import TestClient

    from prime_rl_b200.dashboard import server as dash
    from prime_rl_b200.monitors import FileMonitor
    from prime_rl_b200.orchestrator.orchestrator import trace_record
    from prime_rl_b200.orchestrator.types import Rollout, Turn

    monkeypatch.setattr(dash, "STATE_DIR", tmp_path / "state")
    monkeypatch.setattr(dash, "DIRS_FILE", tmp_path / "state" / "dirs.json")
    run = tmp_path / "run"
    run.mkdir()
    (run / "rl.toml").write_text("max_steps = 3\n")
    (run / "trainer.log").write_text("line one\nline two\n")
    orch, trainer = FileMonitor(run, "orchestrator"), FileMonitor(run, "trainer")
    r = Rollout("reverse-text", 3, "g", [Turn([1, 2, 3], [7, 8], [-0.5, -1.25], finish_reason="stop")], reward=0.75,
                advantage=0.25)
    orch.log_trace(trace_record(r, step=4))
    orch.finalize()
    trainer.log_annotations([{"trace_id": r.trace_id, "branch_index": 0, "step": 4,
                              "logprobs": [0, 0, 0, -0.4, -1.5], "entropy": [0, 0, 0, 0.9, 1.1],
                              "loss_mask": [False] * 3 + [True] * 2}], "trainer")
    client = TestClient(dash.build_app([str(run)]))
    rows = client.get("/api/runs/0/traces").json()
    assert len(rows) == 1 and rows[0]["trace_id"] == r.trace_id and rows[0]["tokens"] == 2 and rows[0]["step"] == 4
    full = client.get(f"/api/runs/0/traces/{r.trace_id}").json()
    assert full["turns"][0]["completion_ids"] == [7, 8] and full["annotations"][0]["logprobs"][3] == -0.4
    assert client.get("/api/runs/0/traces/nope").status_code == 404
    assert "rl.toml" in client.get("/api/runs/0/configs").json()
    assert "line two" in client.get("/api/runs/0/logs").json()["trainer.log"]
    other = tmp_path / "run2"
    other.mkdir()
    assert str(other.resolve()) in client.post("/api/view", json={"path": str(other)}).json()["runs"]
    assert "Traces" in client.get("/").text


def test_dashboard_episode_browser_queries(tmp_path, monkeypatch):
    """Filtered / sorted pages, histogram, per-step series, rollout groups, per-episode timeline with the
    trainer's annotations, metric down-sampling, paged log reads and the run-list event stream."""
    from fastapi.testclient import TestClient

    from prime_rl_b200.dashboard import server as dash
    from prime_rl_b200.monitors import FileMonitor
    from prime_rl_b200.orchestrator.orchestrator import trace_record
    from prime_rl_b200.orchestrator.types import Rollout, Turn

    monkeypatch.setattr(dash, "STATE_DIR", tmp_path / "state")
    monkeypatch.setattr(dash, "DIRS_FILE", tmp_path / "state" / "dirs.json")
    run = tmp_path / "run"
    run.mkdir()
    (run / "logs").mkdir()
    (run / "logs" / "trainer.log").write_text("".join(f"line {i}\n" for i in range(1000)))
    orch, trainer = FileMonitor(run, "orchestrator", chunk_size=4), FileMonitor(run, "trainer")
    made = []
    for step in (1, 2, 3):
        for task in range(2):
            for sample in range(3):
                rew = float((task + sample + step) % 2)
                r = Rollout("rev" if task == 0 else "math", task, f"g{step}-{task}",
                            [Turn([1, 2], [5, 6, 7][:1 + sample], [-0.5] * (1 + sample), finish_reason="stop")],
                            reward=rew, advantage=rew - 0.5, policy_version=step - 1)
                orch.log_trace(trace_record(r, step=step))
                made.append(r)
        trainer.log({"loss": 1.0 / step}, step)
    orch.finalize()
    last = made[-1]
    trainer.log_annotations([{"trace_id": last.trace_id, "branch_index": 0, "step": 3,
                              "logprobs": [0, 0, -0.4, -0.6, -0.5], "entropy": [0, 0, 1.0, 1.0, 1.0],
                              "loss_mask": [False, False, True, True, True]}], "trainer")
    trainer.finalize()
    client = TestClient(dash.build_app([str(run)]))
    page = client.get("/api/runs/0/episodes", params={"limit": 5, "sort": "reward"}).json()
    assert page["total"] == 18 and len(page["rows"]) == 5 and page["rows"][0]["reward"] == 1.0
    assert page["envs"] == ["math", "rev"] and page["steps"] == [1, 3]
    only = client.get("/api/runs/0/episodes", params={"step": 2, "env": "rev", "min_reward": 0.5}).json()
    assert only["total"] == sum(1 for r in made if r.env_name == "rev" and r.reward >= 0.5 and r.policy_version == 1)
    assert all(r["step"] == 2 and r["env"] == "rev" and r["reward"] >= 0.5 for r in only["rows"])
    assert client.get("/api/runs/0/episodes", params={"offset": 15, "limit": 10}).json()["rows"].__len__() == 3
    h = client.get("/api/runs/0/episodes/histogram", params={"bins": 2}).json()
    assert h["n"] == 18 and sum(h["counts"]) == 18 and len(h["counts"]) == 2
    ser = client.get("/api/runs/0/episodes/series").json()
    assert [p["step"] for p in ser] == [1, 2, 3] and all(p["count"] == 6 for p in ser)
    groups = client.get("/api/runs/0/rollouts", params={"step": 3}).json()
    assert groups["total"] == 2 and all(g["size"] == 3 for g in groups["groups"])
    assert {g["group_id"] for g in groups["groups"]} == {"g3-0", "g3-1"} and groups["groups"][0]["reward_spread"] == 1.0
    tl = client.get(f"/api/runs/0/episodes/{last.trace_id}/timeline").json()
    turn = tl["turns"][0]
    assert turn["completion_tokens"] == 3 and turn["loss_tokens"] == 3
    assert turn["trainer_logprob_sum"] == pytest.approx(-1.5) and turn["mean_abs_gap"] == pytest.approx(0.2 / 3)
    assert turn["mismatch_kl"] > 0
    pts = client.get("/api/runs/0/series", params={"key": "loss", "points": 2}).json()
    assert len(pts) == 2 and pts[0]["count"] == 2
    files = client.get("/api/runs/0/logfiles").json()
    assert files[0]["name"] == "logs/trainer.log"
    tail = client.get("/api/runs/0/log", params={"name": "logs/trainer.log", "lines": 3}).json()
    assert tail["text"].split("\n")[-2:] == ["line 999", ""] and tail["end"] == tail["size"]
    head = client.get("/api/runs/0/log", params={"name": "logs/trainer.log", "offset": 0, "lines": 2}).json()
    assert head["text"] == "line 0\nline 1"
    assert client.get("/api/runs/0/log", params={"name": "../secret.log"}).status_code in (403, 404)
    ev = client.get("/api/view/events", params={"once": True}).text
    assert ev.startswith("event: runs") and str(run) in ev
    # the index only reads what is new
    orch2 = FileMonitor(run, "orchestrator2", chunk_size=1)
    orch2.log_trace(trace_record(made[0], step=9))
    orch2.finalize()
    assert client.get("/api/runs/0/episodes").json()["total"] == 19


def test_nccl_transport_probe_with_a_fake_nvml():
    from prime_rl_b200.utils import nccl

    class FakeNVML:
        def __init__(self, links):
            self.links, self.shutdowns = links, 0

        def nvmlInit(self): pass
        def nvmlShutdown(self): self.shutdowns += 1
        def nvmlDeviceGetCount(self): return len(self.links)
        def nvmlDeviceGetHandleByIndex(self, i): return i

        def nvmlDeviceGetNvLinkState(self, h, link):
            if link >= len(self.links[h]):
                raise RuntimeError("not supported")
            return self.links[h][link]

    with_links, without = FakeNVML([[0, 1], [0, 0]]), FakeNVML([[0, 0], []])
    assert nccl.nvlink_present(with_links) is True and nccl.nvlink_present(without) is False
    env = {}
    assert nccl.configure_nccl_transports(with_links, env) is False and env == {}
    assert nccl.configure_nccl_transports(without, env) is True
    assert env == {"NCCL_P2P_DISABLE": "1", "NCCL_SHM_DISABLE": "1"} and without.shutdowns == 2
    env = {"NCCL_P2P_DISABLE": "0", "NCCL_SHM_DISABLE": "0"}
    assert nccl.configure_nccl_transports(without, env) is False and env["NCCL_P2P_DISABLE"] == "0"


def test_rl_launcher_prepares_one_env_server_per_source(tmp_path):
    """With ``spawn_env_servers`` every train / eval source gets an env-server config at its derived address and
    the orchestrator's source is re-pointed at it; explicit ``serve.address`` sources stay externally managed."""
    import json

    from prime_rl_b200.configs.evals import EnvServerConfig
    from prime_rl_b200.configs.rl import RLConfig
    from prime_rl_b200.entrypoints.rl import prepare_env_servers

    cfg = RLConfig.model_validate({"output_dir": str(tmp_path), "orchestrator": {
        "spawn_env_servers": True, "env_server_base_port": 6100,
        "train": {"source": [{"id": "reverse-text"}, {"id": "copy", "name": "cp", "serve": {"address": "http://envs:9"}}]},
        "eval": {"source": [{"env": {"taskset": {"id": "copy"}}, "name": "held-out"}]}}})
    o = cfg.orchestrator
    assert o.env_addresses == {("train", "reverse-text"): "http://127.0.0.1:6100", ("train", "cp"): "http://envs:9",
                               ("eval", "held-out"): "http://127.0.0.1:6102"}
    servers = prepare_env_servers(cfg, tmp_path)
    assert [s[0] for s in servers] == ["env-train-reverse-text", "env-eval-held-out"]
    assert o.train.source[0].id == "remote" and o.train.source[0].args == {"base_url": "http://127.0.0.1:6100"}
    assert o.train.source[1].id == "copy"                                    # externally managed: left alone
    spec = EnvServerConfig.model_validate(json.loads((tmp_path / "envs" / "eval-held-out.json").read_text()))
    assert spec.env.id == "copy" and spec.serve.port == 6102 and spec.env.resolved_name == "held-out"


def test_platform_monitor_uploads_through_a_background_queue(monkeypatch):
    """Registration, per-step metric rows, sampled traces every 10th step as one file, the terminal status, retry
    of a failed request, attach through $RUN_ID and the disabled mode; the HTTP side is an in-process fake."""
    import httpx

    from prime_rl_b200.configs.monitors import PrimeMonitorConfig
    from prime_rl_b200.monitors.prime import PrimeMonitor, encode_samples, resolve_base_url, sanitize

    calls, fail_once = [], {"left": 1}

    def handler(request: httpx.Request) -> httpx.Response:
        path = request.url.path
        if path.endswith("/metrics") and fail_once["left"]:
            fail_once["left"] -= 1
            return httpx.Response(503)
        calls.append((path, dict(request.url.params), request.content))
        if path == "/runs":
            return httpx.Response(200, json={"id": "run-7", "url": "https://tracker/run-7"})
        return httpx.Response(200, json={})

    monkeypatch.delenv("RUN_ID", raising=False)
    monkeypatch.delenv("PRIME_RUNS_MODE", raising=False)
    client = httpx.Client(transport=httpx.MockTransport(handler), base_url="https://tracker")
    mon = PrimeMonitor(PrimeMonitorConfig(run_name="exp"), "orchestrator",
                       {"model": {"name": "tiny"}, "batch_size": 8, "train": {"source": [{"id": "reverse"}]}},
                       client=client, finish_timeout=20.0)
    assert mon.run_id == "run-7" and not mon.attached
    mon.log({"reward": 0.5, "bad": float("nan"), "n": 3}, step=10)
    for i in range(3):
        mon.log_trace({"step": 10, "trace_id": f"t{i}", "turns": [[1, 2], [3]], "reward": 1.0})
    mon.log_trace({"step": 11, "trace_id": "x", "reward": 0.0})       # off the cadence: not shipped
    mon.log({"reward": 0.75}, step=11)
    mon.finalize()
    paths = [c[0] for c in calls]
    assert paths[0] == "/runs" and json.loads(calls[0][2])["model"] == "tiny"
    rows = [json.loads(c[2]) for c in calls if c[0].endswith("/metrics")]
    assert [r["step"] for r in rows] == [10, 11] and rows[0]["metrics"] == {"reward": 0.5, "n": 3}   # 503 was retried
    samples = [c for c in calls if c[0].endswith("/samples")]
    assert len(samples) == 1 and samples[0][1] == {"step": "10", "count": "3"}
    import pyarrow.parquet as pq
    import io

    table = pq.read_table(io.BytesIO(samples[0][2]))
    assert table.num_rows == 3 and json.loads(table.column("turns")[0].as_py()) == [[1, 2], [3]]
    assert paths[-1].endswith("/status") and json.loads(calls[-1][2])["status"] == "completed"

    # attach: no registration, and a crash is left to the launcher
    calls.clear()
    monkeypatch.setenv("RUN_ID", "managed-1")
    att = PrimeMonitor(PrimeMonitorConfig(), "orchestrator", {}, client=client, finish_timeout=20.0)
    assert att.attached and att.run_id == "managed-1"
    att.finalize("crashed")
    assert not any(c[0].endswith("/status") or c[0] == "/runs" for c in calls)
    monkeypatch.delenv("RUN_ID")

    monkeypatch.setenv("PRIME_RUNS_MODE", "disabled")
    off = PrimeMonitor(PrimeMonitorConfig(), "trainer", {})
    off.log({"a": 1}, 0)
    off.finalize()
    monkeypatch.delenv("PRIME_RUNS_MODE")
    with pytest.raises(RuntimeError, match="PRIME_API_KEY"):
        monkeypatch.delenv("PRIME_API_KEY", raising=False)
        PrimeMonitor(PrimeMonitorConfig(), "trainer", {})
    monkeypatch.setenv("PRIME_API_BASE", "https://api.example/api/v1/rft/")
    assert resolve_base_url("https://unused") == "https://api.example/api/v1"
    assert sanitize({"a": float("inf"), "b": True, "c": [1]}) == ({"b": 1}, ["a", "c"])
    assert encode_samples([{"a": 1}])[1] in ("application/vnd.apache.parquet", "application/x-ndjson")
