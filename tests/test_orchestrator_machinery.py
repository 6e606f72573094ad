"""Scheduling rules of the orchestrator on fakes (CPU, asyncio only): pending weight updates stop scheduling and
cut hopeless train groups, admissions are capped per burst window, evals take priority while queued and
assemble into epochs, a run that admits nothing for ten batch-equivalents aborts, engine metrics roll up.
"""

import asyncio
import time
from types import SimpleNamespace

import pytest

from prime_rl_b200.configs.orchestrator import ConcurrencyConfig, OrchestratorConfig
from prime_rl_b200.orchestrator.concurrency import ConcurrencyController
from prime_rl_b200.orchestrator.eval_sink import EvalSink, EvalWork
from prime_rl_b200.orchestrator.inference_metrics import InferenceMetrics
from prime_rl_b200.orchestrator.orchestrator import (Dispatcher, DispatcherMode, Source, TrainSink, WeightWatcher,
                                                     min_fresh_version)
from prime_rl_b200.orchestrator.types import Policy, Rollout, Turn


class SlowEnv:
    """Episodes that finish when the test says so."""

    def __init__(self, name="slow", num_tasks=1000):
        self.name, self.num_tasks = name, num_tasks
        self.release = asyncio.Event()
        self.started = 0

    async def rollout(self, client, task_id, sampling, policy_version, group_id):
        self.started += 1
        await self.release.wait()
        t = Turn([1, 2], [3], [-0.1])
        return Rollout(self.name, task_id, group_id, [t], reward=float(task_id % 2), policy_version=policy_version)


class NullAlgo:
    action_loss_type = "rl"
    config = SimpleNamespace(sampling=SimpleNamespace(source="policy"))

    async def finalize_episode(self, r):
        return None


def _dispatcher(env, group_size=2, limit=64, **kw):
    ctrl = ConcurrencyController(ConcurrencyConfig(initial_inflight=limit, max_inflight=limit), group_size)
    policy = Policy()
    src = Source(env, NullAlgo(), group_size, SimpleNamespace(temperature=1.0), 1.0)
    return Dispatcher([src], client=None, policy=policy, controller=ctrl, **kw), policy, src


def test_min_fresh_version_matches_the_shipping_rule():
    # batch `step` trains on policy step - 1; an episode may lag it by max_off_policy_steps versions
    assert min_fresh_version(10, 8) == 1 and min_fresh_version(3, 0) == 2


def test_pending_weight_update_stops_scheduling_and_cuts_hopeless_groups():
    async def go():
        env = SlowEnv()
        d, policy, _ = _dispatcher(env, max_off_policy_steps=1, min_burst=100)
        d.controller.limit = 8
        runner = asyncio.create_task(d.run())
        await asyncio.sleep(0.05)
        old = set(d.groups)                                   # launched at policy version 0
        assert len(old) == 4 and all(m.policy_version_at_start == 0 for m in d.groups.values())
        policy.version = 3
        d.controller.limit = 16
        await asyncio.sleep(0.05)                             # newer groups join at version 3
        fresh = set(d.groups) - old
        assert fresh
        d.progress_step = 4                                   # batch 4 trains on v3: versions < 2 can never ship
        cancelled = await d.on_version_pending(3)
        assert d.policy_update_pending and cancelled == sum(2 for _ in old)
        await asyncio.sleep(0.05)
        assert not (set(d.groups) & old) and fresh <= set(d.groups)
        launched = d.stats["groups_launched"]
        await asyncio.sleep(0.05)
        assert d.stats["groups_launched"] == launched         # nothing is scheduled while the update is pending
        await d.on_new_version(3)
        env.release.set()
        await asyncio.sleep(0.05)
        assert d.stats["groups_launched"] > launched
        lost = []
        while not d.out_q.empty():
            item = d.out_q.get_nowait()
            if isinstance(item, tuple):
                lost.append(item)
        assert len([x for x in lost if x[0] == "cancel" and x[2] == "train"]) == cancelled
        await d.stop()
        runner.cancel()

    asyncio.run(go())


def test_admissions_are_capped_per_burst_window():
    async def go():
        env = SlowEnv()
        d, _, _ = _dispatcher(env, group_size=1, limit=1000, min_burst=5, admission_window_s=3600.0)
        for _ in range(400):                                  # far more scheduling passes than the cap allows
            await d.fill_inflight()
        cap = max(5, 1000 // 10)
        assert d.stats["groups_launched"] == cap              # one window's cap, not the whole budget of 1000
        assert d.admission_budget() == 0
        d._window_start -= 7200.0                             # the window has passed
        for _ in range(400):
            await d.fill_inflight()
        assert d.stats["groups_launched"] == 2 * cap
        env.release.set()
        await d.stop()

    asyncio.run(go())


def test_eval_work_takes_priority_and_assembles_into_an_epoch():
    async def go():
        train_env, eval_env = SlowEnv("train"), SlowEnv("held-out", num_tasks=3)
        d, policy, _ = _dispatcher(train_env, group_size=2, limit=8, min_burst=100)
        eval_src = Source(eval_env, None, 2, SimpleNamespace(temperature=0.0), 1.0)
        sink = EvalSink()
        sink.expect("held-out", 5, num_examples=3, group_size=2)
        d.dispatch_allowed.clear()                            # evals ignore the train gate
        d.request_eval([EvalWork(eval_src, t, 5) for t in range(3)])
        assert d.mode is DispatcherMode.PREFER_EVAL
        runner = asyncio.create_task(d.run())
        await asyncio.sleep(0.05)
        assert eval_env.started == 6 and train_env.started == 0
        assert d.mode is DispatcherMode.PREFER_TRAIN          # queue drained -> back to train work
        d.dispatch_allowed.set()
        await asyncio.sleep(0.05)
        assert train_env.started == 2                         # 8 slots - 6 eval episodes
        eval_env.release.set()
        rows = []
        for _ in range(6):
            r = await asyncio.wait_for(d.out_q.get(), 1.0)
            assert r.info["_kind"] == "eval" and r.info["_eval_step"] == 5
            row = sink.add(r, 5)
            if row:
                rows.append(row)
        assert len(rows) == 1
        row = rows[0]
        assert row["env"] == "held-out" and row["rollouts"] == 6 and row["num_examples"] == 3
        assert row["reward/mean"] == pytest.approx(2 / 6) and row["pass@2"] == pytest.approx(1 / 3)
        train_env.release.set()
        await d.stop()
        runner.cancel()

    asyncio.run(go())


def test_eval_epoch_counts_failures_and_can_be_superseded():
    sink = EvalSink()
    sink.expect("e", 2, num_examples=2, group_size=2)
    t = Turn([1], [2, 3], [-0.1, -0.2])
    assert sink.add(Rollout("e", 0, "g", [t], reward=1.0, policy_version=2), 2) is None
    assert sink.fail("e", 2) is None
    assert sink.cancel("e", 2) is None
    row = sink.add(Rollout("e", 1, "h", [t], reward=0.0, policy_version=2), 2)
    assert row["failed"] == 1 and row["cancelled"] == 1 and row["rollouts"] == 2 and row["completion_len/mean"] == 2
    sink.expect("e", 4, 4, 1)
    sink.add(Rollout("e", 0, "g", [t], reward=1.0, policy_version=4), 4)
    closed = sink.abandon(6)                                  # a newer eval begins: close what is there
    assert len(closed) == 1 and closed[0]["cancelled"] == 3 and not sink.epochs


def test_train_sink_aborts_after_ten_batch_equivalents_without_payload():
    cfg = OrchestratorConfig(batch_size=4, group_size=2, max_off_policy_steps=0)
    policy = Policy(version=5)
    sink = TrainSink(cfg, policy)
    src = Source(SlowEnv(), NullAlgo(), 2, None, 1.0)
    t = Turn([1], [2], [-0.1])

    async def stale_group(i):
        for _ in range(2):
            r = Rollout("slow", i, f"g{i}", [t], reward=0.0, policy_version=0)      # 5 versions behind, bound 0
            r.info["_source"] = src
            await sink.add(r)

    async def go():
        for i in range(19):                                   # 38 rollouts = 9.5 batches of 4
            await stale_group(i)
        assert sink.stats["groups_dropped_stale"] == 19
        with pytest.raises(RuntimeError, match="zero-output"):
            await stale_group(19)

    asyncio.run(go())


def test_weight_watcher_brackets_the_update_with_the_dispatcher_hooks():
    calls = []

    class FakeDispatcher:
        async def on_version_pending(self, step):
            calls.append(("pending", step))
            return 3

        async def on_new_version(self, step):
            calls.append(("new", step))

    class FakeReceiver:
        def pending_step(self, after):
            return 7 if after < 7 else None

        async def receive(self, step):
            calls.append(("receive", step))

    policy = Policy()
    w = WeightWatcher(FakeReceiver(), policy, FakeDispatcher())
    assert asyncio.run(w.sync_once())
    assert calls == [("pending", 7), ("receive", 7), ("new", 7)] and policy.version == 8
    assert w.stats["episodes_cancelled_stale"] == 3


def test_inference_metrics_rates_and_histogram():
    m = InferenceMetrics()
    m.ingest([{"vllm:kv_cache_usage_perc": 0.2, "vllm:num_requests_running": 10, "vllm:generation_tokens_total": 100},
              {"vllm:kv_cache_usage_perc": 0.85, "vllm:num_requests_running": 30, "vllm:generation_tokens_total": 50}])
    time.sleep(0.05)
    m.ingest([{"vllm:kv_cache_usage_perc": 0.4, "vllm:num_requests_running": 20, "vllm:generation_tokens_total": 400},
              {"vllm:kv_cache_usage_perc": 0.95, "vllm:num_requests_running": 40, "vllm:generation_tokens_total": 20}])
    snap = m.snapshot()
    assert snap["inference/kv_usage/max"] == pytest.approx(0.95) and snap["inference/running/mean"] == pytest.approx(25)
    # engine 0 produced 300 tokens in the window; engine 1 restarted (its counter fell) and is not counted negative
    assert snap["inference/generation_tokens/per_s"] > 0
    assert snap["inference/generation_tokens/per_s"] * 0.05 <= 300 * 1.01
    assert sum(v for k, v in snap.items() if k.startswith("inference/kv_usage_hist/")) == pytest.approx(1.0)
    assert m.snapshot()["inference/scrapes"] == 0.0           # a new window began
