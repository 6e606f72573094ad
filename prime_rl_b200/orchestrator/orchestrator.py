"""Asynchronous RL orchestrator: schedules environment episodes against the inference pool,
scores completed groups, packs samples into per-rank micro-batches for the trainer and
relays new policy versions into the engines.

Asynchrony contract (reference: src/prime_rl/orchestrator/orchestrator.py:95-98, :634-652):
batch ``step`` is shipped only once the engines run policy version >= ``step - 1 -
TARGET_LAG``; rollouts generated more than ``max_off_policy_steps`` versions ago are dropped.

Parts:
  Dispatcher     keeps up to the controller's limit of episodes in flight, one group per task; train and
                 eval work share it (PREFER_TRAIN / PREFER_EVAL), admissions are rate-limited per burst
                 window, scheduling stops while a weight update is pending and train groups that could
                 never ship inside ``max_off_policy_steps`` are cancelled before the engines pause
  TrainSink      groups -> advantages -> samples -> pending batch (stale / zero-advantage pruning); aborts
                 after 10 batch-equivalents of finalized rollouts that admitted nothing
  EvalSink       (eval_sink.py) eval episodes -> per (env, step) epochs -> eval metrics
  WeightWatcher  polls ``broadcasts/`` for offered versions and runs the receiver handshake
  Orchestrator   main loop, eval triggering, engine metrics, event-loop lag, checkpoints
"""

from __future__ import annotations

import asyncio
import enum
import os
import random
import threading
import time
import uuid
from collections import defaultdict
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .. import monitors as monitors_mod
from ..configs.orchestrator import OrchestratorConfig
from ..trainer.batch import prepare_batch
from ..transports.batch import setup_batch_sender
from ..transports.weights import WeightReceiver
from ..utils.logger import get_logger
from ..utils.pathing import get_ckpt_dir, get_step_path, latest_step
from .algo import setup_algorithm
from .clients import AdminPlane, InferenceClient
from .concurrency import ConcurrencyController
from .envs import load_environment
from .eval_sink import EvalSink, EvalWork
from .inference_metrics import InferenceMetrics
from .types import Policy, Rollout

TARGET_LAG = 1
MAX_EMPTY_BATCHES = 10
MAX_ZERO_OUTPUT_BATCH_EQUIVALENTS = 10      # finalized rollouts worth this many batches without any admitted payload
TEARDOWN_TIMEOUT_S = 300.0                  # a shutdown that hangs longer than this ends the process


def min_fresh_version(step: int, max_off_policy_steps: int) -> int:
    """Oldest dispatch version whose episodes can still train in batch ``step`` (which trains on policy
    ``step - 1``); anything older would ship beyond ``max_off_policy_steps``."""
    return (step - 1) - max_off_policy_steps


class DispatcherMode(enum.Enum):
    PREFER_TRAIN = "train"
    PREFER_EVAL = "eval"


@dataclass
class GroupMeta:
    kind: str                       # "train" | "eval"
    env_name: str
    policy_version_at_start: int
    live: bool                      # sampled from the live policy (frozen-sourced groups never go stale)
    size: int
    eval_step: int = -1
    tasks: list = field(default_factory=list)


@dataclass
class Source:
    env: object
    algo: object
    group_size: int
    sampling: object
    ratio: float
    next_task: int = 0
    gates: list = field(default_factory=list)
    sampler: object = None          # orchestrator/curriculum.py task sampler (None: round robin)


class Dispatcher:
    """Fills the in-flight budget with group episodes; finished rollouts go to ``out_q`` as ``Rollout``
    objects, lost ones as ``("cancel" | "fail", group_id, kind, env_name, eval_step, detail)`` tuples.

    Scheduling rules (reference: src/prime_rl/orchestrator/dispatcher.py:276-283 burst budget, :363-401
    pending weight update, :407-440 modes):
      * at most ``max(min_burst, max_inflight // 10)`` group admissions per ``admission_window_s``;
      * ``PREFER_EVAL`` while eval work is queued (evals ignore the train dispatch gate), back to
        ``PREFER_TRAIN`` once the eval queue drained;
      * nothing is scheduled between ``on_version_pending`` and ``on_new_version``.
    """

    def __init__(self, sources: list[Source], client: InferenceClient, policy: Policy,
                 controller: ConcurrencyController, seed: int = 0, tasks_per_minute: int | None = None,
                 max_off_policy_steps: int = 8, min_burst: int = 4, admission_window_s: float = 1.0):
        self.sources, self.client, self.policy, self.controller = sources, client, policy, controller
        self.out_q: asyncio.Queue = asyncio.Queue()
        self.inflight: dict[asyncio.Task, str] = {}
        self.groups: dict[str, GroupMeta] = {}
        self.rng = random.Random(seed)
        self.paused = asyncio.Event()
        self.paused.set()
        self.dispatch_allowed = asyncio.Event()          # the orchestrator's gate on *train* scheduling
        self.dispatch_allowed.set()
        self.scheduling_lock = asyncio.Lock()
        self.stopped = False
        self.mode = DispatcherMode.PREFER_TRAIN
        self.eval_queue: list[EvalWork] = []
        self.policy_update_pending = False
        self.max_off_policy_steps = max_off_policy_steps
        self.progress_step = 0                           # batch the orchestrator is collecting (set by its loop)
        self.tasks_per_minute = tasks_per_minute
        self.min_burst, self.admission_window_s = min_burst, admission_window_s
        self._window_start, self._admissions = time.monotonic(), 0
        self._last_launch = 0.0
        self.stats = defaultdict(int)

    # ------------------------------------------------------------------ admission
    def admission_budget(self) -> int:
        """Group admissions still allowed in the current burst window."""
        now = time.monotonic()
        if now - self._window_start >= self.admission_window_s:
            self._window_start, self._admissions = now, 0
        cap = max(self.min_burst, (self.controller.max or self.controller.limit) // 10)
        return cap - self._admissions

    def switch_mode(self, mode: DispatcherMode, reason: str = "") -> None:
        if mode != self.mode:
            self.mode = mode
            self.stats[f"mode_switches_to_{mode.value}"] += 1
            get_logger().info(f"dispatcher prefers {mode.value} work now ({reason})")

    def request_eval(self, work: list[EvalWork]) -> None:
        """Queues eval examples and gives them priority over train scheduling until they are dispatched."""
        self.eval_queue.extend(work)
        if self.eval_queue:
            self.switch_mode(DispatcherMode.PREFER_EVAL, "an eval was triggered")

    def _pick(self) -> Source:
        total = sum(s.ratio for s in self.sources)
        x = self.rng.random() * total
        for s in self.sources:
            x -= s.ratio
            if x <= 0:
                return s
        return self.sources[-1]

    async def _episode(self, src: Source, task_id: int, group_id: str, kind: str, eval_step: int) -> None:
        version = self.policy.version
        try:
            r: Rollout = await src.env.rollout(self.client, task_id, src.sampling, version, group_id)
            if kind == "train":
                await src.algo.finalize_episode(r)
            r.info["_source"], r.info["_kind"], r.info["_eval_step"] = src, kind, eval_step
            await self.out_q.put(r)
            self.stats["episodes_ok"] += 1
        except asyncio.CancelledError:
            self.stats["episodes_cancelled"] += 1
            await self.out_q.put(("cancel", group_id, kind, src.env.name, eval_step, ""))
            raise
        except Exception as e:
            self.stats["episodes_failed"] += 1
            await self.out_q.put(("fail", group_id, kind, src.env.name, eval_step, repr(e)))
        finally:
            self.controller.on_episode_done()

    def _launch(self, src: Source, task_id: int, kind: str, eval_step: int = -1) -> None:
        gid = uuid.uuid4().hex
        live = getattr(getattr(src.algo, "config", None), "sampling", None) is None or \
            getattr(src.algo.config.sampling, "source", "policy") == "policy"
        meta = GroupMeta(kind, getattr(src.env, "name", "env"), self.policy.version, live, src.group_size, eval_step)
        self.groups[gid] = meta
        for _ in range(src.group_size):
            t = asyncio.create_task(self._episode(src, task_id, gid, kind, eval_step))
            self.inflight[t] = gid
            meta.tasks.append(t)
            t.add_done_callback(self._on_task_done)
        self._admissions += 1
        self.stats[f"{kind}_groups_launched"] += 1
        self.stats["groups_launched"] += 1

    def _on_task_done(self, t: asyncio.Task) -> None:
        gid = self.inflight.pop(t, None)
        meta = self.groups.get(gid)
        if meta is not None and all(x.done() for x in meta.tasks):
            self.groups.pop(gid, None)

    def _launch_train_group(self) -> None:
        src = self._pick()
        if src.sampler is not None:
            task_id = src.sampler.sample()
            src.next_task = getattr(src.sampler, "next", src.next_task)
        else:
            task_id = src.next_task % max(1, getattr(src.env, "num_tasks", 1 << 30))
            src.next_task += 1
        self._launch(src, task_id, "train")

    async def fill_inflight(self) -> bool:
        """Schedules at most one group; returns whether it did."""
        if self.policy_update_pending or self.admission_budget() <= 0:
            return False
        async with self.scheduling_lock:
            if self.policy_update_pending:
                return False
            room = self.controller.limit - len(self.inflight)
            if self.mode == DispatcherMode.PREFER_EVAL:
                if not self.eval_queue:
                    self.switch_mode(DispatcherMode.PREFER_TRAIN, "the eval queue drained")
                    return False
                work = self.eval_queue[0]
                if room < work.source.group_size:
                    return False
                self.eval_queue.pop(0)
                self._launch(work.source, work.task_id, "eval", work.step)
                return True
            if not self.dispatch_allowed.is_set() or not self.sources:
                return False
            if room < min(s.group_size for s in self.sources):
                return False
            if self.tasks_per_minute:
                wait = 60.0 / self.tasks_per_minute - (time.monotonic() - self._last_launch)
                if wait > 0:
                    await asyncio.sleep(wait)
            self._launch_train_group()
            self._last_launch = time.monotonic()
            return True

    async def run(self) -> None:
        while not self.stopped:
            await self.paused.wait()
            if await self.fill_inflight():
                await asyncio.sleep(0)
            else:
                await asyncio.sleep(0.005)

    # ------------------------------------------------------------------ weight updates
    async def drop_group(self, gid: str, reason: str) -> int:
        meta = self.groups.get(gid)
        if meta is None:
            return 0
        n = 0
        for t in meta.tasks:
            if not t.done():
                t.cancel()
                n += 1
        self.stats[f"groups_dropped_{reason}"] += 1
        return n

    async def on_version_pending(self, step: int) -> int:
        """A weight update is about to be applied: stop scheduling, and cancel live-policy train groups that
        started before ``min_fresh_version`` of the batch being collected (they could only ship beyond
        ``max_off_policy_steps``). Runs before the engines are paused, so the aborts are processed while the
        engines still step. Returns the number of cancelled episodes."""
        self.policy_update_pending = True
        async with self.scheduling_lock:        # a scheduling pass that began before the flag finishes first
            pass
        oldest = min_fresh_version(self.progress_step, self.max_off_policy_steps)
        cancelled = 0
        for gid, meta in list(self.groups.items()):
            if meta.kind == "train" and meta.live and meta.policy_version_at_start < oldest:
                cancelled += await self.drop_group(gid, "stale")
        if cancelled:
            get_logger().warning(f"cancelled {cancelled} train episodes past max_off_policy_steps="
                                 f"{self.max_off_policy_steps}; consider raising it")
        return cancelled

    async def on_new_version(self, step: int) -> None:
        self.policy_update_pending = False

    def cancel_newest(self, n: int) -> None:
        for t in list(self.inflight)[-n:]:
            t.cancel()

    async def stop(self) -> None:
        self.stopped = True
        self.paused.set()
        for t in list(self.inflight):
            t.cancel()
        await asyncio.gather(*list(self.inflight), return_exceptions=True)


class TrainSink:
    """Collects rollouts into groups, scores complete groups and accumulates the pending batch."""

    def __init__(self, config: OrchestratorConfig, policy: Policy):
        self.config, self.policy = config, policy
        self.groups: dict[str, list[Rollout]] = defaultdict(list)
        self.dead_groups: set[str] = set()
        self.pending: list[tuple[Rollout, list]] = []     # (rollout, samples)
        self.stats = defaultdict(float)
        self.zero_output_units = 0            # finalized rollouts (or tokens) since the last admitted payload
        self._reported_windows = 0

    def cancel(self, group_id: str) -> None:
        lost = self.groups.pop(group_id, None)
        if group_id not in self.dead_groups:
            self._record_zero_output(lost or [], owed=1)
        self.dead_groups.add(group_id)

    def _record_zero_output(self, group: list, owed: int) -> None:
        """A group ended without contributing anything trainable. After MAX_ZERO_OUTPUT_BATCH_EQUIVALENTS
        batches' worth of such rollouts in a row the run is aborted: the curriculum gates, the task difficulty
        or staleness drops are eating everything (reference: src/prime_rl/orchestrator/train_sink.py:334-363)."""
        c = self.config
        if c.batch_size is not None:
            self.zero_output_units += len(group) or owed
            target = c.batch_size
        else:
            self.zero_output_units += sum(r.num_total_tokens for r in group) or c.seq_len * owed
            target = c.token_batch_size
        windows = self.zero_output_units // max(1, target)
        if windows > self._reported_windows:
            self._reported_windows = windows
            get_logger().warning(f"no admitted train payload after {self.zero_output_units} finalized units "
                                 f"({windows}/{MAX_ZERO_OUTPUT_BATCH_EQUIVALENTS} batch equivalents)")
            if windows >= MAX_ZERO_OUTPUT_BATCH_EQUIVALENTS:
                raise RuntimeError(f"{windows} consecutive zero-output batch equivalents: check the curriculum "
                                   "admission policy, task difficulty and staleness drops")

    def _admitted(self) -> None:
        self.zero_output_units, self._reported_windows = 0, 0

    async def add(self, r: Rollout) -> None:
        if r.group_id in self.dead_groups:
            return
        src: Source = r.info["_source"]
        g = self.groups[r.group_id]
        g.append(r)
        if len(g) >= src.group_size:
            del self.groups[r.group_id]
            await self._process_group(g, src)

    async def _process_group(self, group: list[Rollout], src: Source) -> None:
        oldest = min(r.policy_version for r in group)
        if self.policy.version - oldest > self.config.max_off_policy_steps:
            self.stats["groups_dropped_stale"] += 1
            self._record_zero_output(group, owed=len(group))
            return
        await src.algo.score_group(group)
        if src.sampler is not None:
            src.sampler.update(group[0].task_id, sum(r.reward for r in group) / len(group))
        advs = [r.advantage or 0.0 for r in group]
        for gate in src.gates:
            if all(gate.reject_min <= a <= gate.reject_max for a in advs):
                self.stats["groups_rejected_by_gate"] += 1
                self._record_zero_output(group, owed=len(group))
                return
        self.stats["groups_scored"] += 1
        before = len(self.pending)
        for r in group:
            self.stats["reward_sum"] += r.reward
            self.stats["reward_n"] += 1
            if src.algo.action_loss_type == "rl" and (r.advantage or 0.0) == 0.0 \
                    and src.algo.observation_weights(r, 0) is None:
                self.stats["rollouts_pruned_zero_adv"] += 1
                continue     # contributes no gradient
            self.pending.append((r, src.algo.to_samples(r)))
        if len(self.pending) > before:
            self._admitted()
        # a group whose rollouts all tied (zero advantage) was scored fine and only carries no signal: that case
        # is bounded by the empty-batch counter of the main loop, not by the zero-output budget

    def sweep_stale(self) -> None:
        keep = []
        for r, s in self.pending:
            if self.policy.version - r.policy_version > self.config.max_off_policy_steps:
                self.stats["rollouts_dropped_stale"] += 1
            else:
                keep.append((r, s))
        self.pending = keep

    def maybe_batch(self) -> list[tuple[Rollout, list]] | None:
        """Cuts a batch of ``batch_size`` traces (or ``token_batch_size`` tokens) when available."""
        self.sweep_stale()
        c = self.config
        if c.batch_size is not None:
            # zero-advantage pruning shrinks groups, so count scored rollouts rather than kept ones
            if len(self.pending) >= c.batch_size or \
                    (self.pending and self.stats["reward_n"] - self.stats["reward_n_at_cut"] >= c.batch_size):
                n = min(len(self.pending), c.batch_size)
                batch, self.pending = self.pending[:n], self.pending[n:]
                self.stats["reward_n_at_cut"] = self.stats["reward_n"]
                return batch
            return None
        tokens, n = 0, 0
        for r, _ in self.pending:
            tokens += r.num_total_tokens
            n += 1
            if tokens >= c.token_batch_size:
                batch, self.pending = self.pending[:n], self.pending[n:]
                return batch
        return None


class WeightWatcher:
    """Polls the broadcast directory; when the trainer offers version N, runs the receiver
    handshake (pause -> acknowledge -> update -> resume) and publishes ``policy.version = N + 1``
    (a batch trained at step N yields policy N + 1; step -1 / 0 seeds version 0)."""

    def __init__(self, receiver: WeightReceiver, policy: Policy, dispatcher: Dispatcher, poll: float = 0.05):
        self.receiver, self.policy, self.dispatcher, self.poll = receiver, policy, dispatcher, poll
        self.last_step = -1
        self.stopped = False
        self.stats = defaultdict(float)

    async def sync_once(self) -> bool:
        step = self.receiver.pending_step(self.last_step)
        if step is None:
            return False
        t0 = time.monotonic()
        # stale work is cut while the engines still step (their aborts need a running engine), and no new
        # rollout may start until the new weights are live
        self.stats["episodes_cancelled_stale"] += await self.dispatcher.on_version_pending(step)
        try:
            await self.receiver.receive(step)
        finally:
            await self.dispatcher.on_new_version(step)
        self.last_step = step
        self.policy.version = step + 1
        self.stats["updates"] += 1
        self.stats["last_update_seconds"] = time.monotonic() - t0
        return True

    async def run(self) -> None:
        while not self.stopped:
            try:
                if not await self.sync_once():
                    await asyncio.sleep(self.poll)
            except asyncio.CancelledError:
                raise


class Orchestrator:
    def __init__(self, config: OrchestratorConfig, *, http_transport=None):
        self.config = config
        self.run_dir = Path(config.output_dir)
        self.logger = get_logger()
        self.policy = Policy()
        self.step = 0
        self.http_transport = http_transport

    async def setup(self) -> "Orchestrator":
        c = self.config
        self.client = InferenceClient(c.model.client, c.model.name, transport=self.http_transport,
                                      return_routed_experts=c.enable_return_routed_experts,
                                      return_sampling_mask=c.train.sampling.truncated)
        self.admin = AdminPlane(c.model.client, transport=self.http_transport)
        self.monitor = monitors_mod.setup(c.monitors, self.run_dir, "orchestrator")
        self.sources = []
        for s in c.train.source:
            algo = setup_algorithm(c.source_algo(s), self.client)
            gates = list((s.curriculum.gates.values()) if s.curriculum else [])
            env = load_environment(s)
            from .curriculum import build_sampler

            sampler = build_sampler(s.curriculum, getattr(env, "num_tasks", 1 << 30)) if s.curriculum else None
            self.sources.append(Source(env, algo, c.source_group_size(s), c.source_sampling(s), s.ratio, gates=gates,
                                       sampler=sampler))
        self.sender = setup_batch_sender(self.run_dir, c.num_train_workers, c.rollout_transport)
        await self.admin.wait_for_ready()
        self.controller = ConcurrencyController(c.concurrency, c.group_size)
        self.dispatcher = Dispatcher(self.sources, self.client, self.policy, self.controller, seed=c.seed,
                                     tasks_per_minute=c.tasks_per_minute, max_off_policy_steps=c.max_off_policy_steps)
        self.sink = TrainSink(c, self.policy)
        # online evals: version-pinned measurements that share the dispatcher with training rollouts
        self.eval_sources: list[tuple[object, Source]] = []
        self.eval_sink = EvalSink()
        self._evaluated_versions: set[int] = set()
        if c.eval is not None:
            for es in c.eval.source:
                sampling = es.sampling if (es.sampling.temperature is not None or es.sampling.max_completion_tokens
                                           or es.sampling.top_p is not None) else c.eval.sampling
                from types import SimpleNamespace

                sp = SimpleNamespace(temperature=sampling.temperature if sampling.temperature is not None else 0.0,
                                     top_p=sampling.top_p if sampling.top_p is not None else 1.0, top_k=sampling.top_k,
                                     max_completion_tokens=sampling.max_completion_tokens,
                                     extra_body=sampling.extra_body)
                src = Source(load_environment(es), None, max(es.group_size, c.eval.group_size), sp, 1.0)
                self.eval_sources.append((es, src))
        self.inference_metrics = InferenceMetrics(c.inference_metrics_roles)
        self.loop_lag = {"max": 0.0, "sum": 0.0, "n": 0}
        wb = c.weight_broadcast
        if wb.type == "p2p":
            # every engine publishes the IPC handles of its parameter storage under the run directory
            await self.admin.init_broadcaster(type="p2p", run_dir=str(self.run_dir),
                                              quantize=getattr(wb, "quantize", None))
        elif wb.type == "nccl":
            await self.admin.init_broadcaster(type="nccl", host=wb.host, port=wb.port,
                                              inference_world_size=wb.inference_world_size, timeout=wb.timeout)
        self.receiver = WeightReceiver(c.weight_broadcast, self.run_dir, self.admin)
        self.watcher = WeightWatcher(self.receiver, self.policy, self.dispatcher)
        self._maybe_resume()
        return self

    # ------------------------------------------------------------------ checkpoint
    def _ckpt_path(self, step: int) -> Path:
        return get_step_path(get_ckpt_dir(self.run_dir), step) / "orchestrator" / "progress.pt"

    def save_ckpt(self, step: int) -> None:
        p = self._ckpt_path(step)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(".tmp")
        state = {"step": step, "policy_version": self.policy.version,
                 "next_task": [s.next_task for s in self.sources],
                 "sampler": [s.sampler.state_dict() if s.sampler is not None else None for s in self.sources],
                 "algo": [s.algo.state_dict() if hasattr(s.algo, "state_dict") else None for s in self.sources]}
        torch.save(state, tmp)
        tmp.replace(p)

    def _maybe_resume(self) -> None:
        c = self.config
        if c.resume is None:
            return
        step = c.resume.step if c.resume.step is not None else latest_step(get_ckpt_dir(self.run_dir))
        if step is None or not self._ckpt_path(step).exists():
            return
        state = torch.load(self._ckpt_path(step), weights_only=False)
        self.step = state["step"] + 1
        for s, sd in zip(self.sources, state.get("sampler", [])):
            if s.sampler is not None and sd is not None:
                s.sampler.load_state_dict(sd)
        for s, nt, a in zip(self.sources, state["next_task"], state["algo"]):
            s.next_task = nt
            if a is not None and hasattr(s.algo, "load_state_dict"):
                s.algo.load_state_dict(a)
        self.watcher.last_step = state["step"] - 1

    # ------------------------------------------------------------------ main loop
    async def _ship(self, batch) -> dict:
        c = self.config
        need = self.step - 1 - TARGET_LAG
        t0 = time.monotonic()
        while self.policy.version < need + 1 and need >= 0:
            await asyncio.sleep(0.01)            # hold the batch until inference caught up
        wait = time.monotonic() - t0
        samples = [s for _, ss in batch for s in ss]
        grid = await asyncio.to_thread(prepare_batch, samples, seq_len=c.seq_len,
                                       num_train_workers=c.num_train_workers,
                                       pad_to_multiple_of=c.pad_to_multiple_of)
        await asyncio.to_thread(self.sender.send, self.step, grid)
        rollouts = [r for r, _ in batch]
        for r in rollouts:                       # one trace record per episode, joined to the trainer's
            self.monitor.log_trace(trace_record(r, self.step))     # annotations by (trace_id, branch_index)
        lag = [self.policy.version - r.policy_version for r in rollouts]
        m = {
            "reward": sum(r.reward for r in rollouts) / len(rollouts),
            "seq_len/mean": sum(r.num_total_tokens for r in rollouts) / len(rollouts),
            "seq_len/max": max(r.num_total_tokens for r in rollouts),
            "batch/rollouts": len(rollouts), "batch/micro_steps": len(grid[0]),
            "off_policy/mean": sum(lag) / len(lag), "off_policy/max": max(lag),
            "time/wait_for_weights": wait, "policy_version": self.policy.version,
            "dispatcher/inflight": len(self.dispatcher.inflight), "dispatcher/limit": self.controller.limit,
            "sink/pending": len(self.sink.pending),
        }
        m.update({f"sink/{k}": v for k, v in self.sink.stats.items() if not k.startswith("reward_")})
        m.update({f"dispatcher/{k}": v for k, v in self.dispatcher.stats.items()})
        m.update({f"watcher/{k}": v for k, v in self.watcher.stats.items()})
        return m

    async def _serve_remaining_weight_updates(self, timeout: float | None = None) -> None:
        """The last batches ship up to ``TARGET_LAG + 1`` trainer steps ahead of the weights. A trainer whose sender
        waits for the receiver's acknowledgement (the in-memory transports) still offers the weights of every step
        but the last one, so the watcher keeps answering until version ``max_steps - 1`` is live; leaving earlier
        would park the trainer in its acknowledgement wait until that times out."""
        c = self.config
        if c.max_steps is None or getattr(c.weight_broadcast, "type", "filesystem") == "filesystem":
            return
        timeout = timeout if timeout is not None else float(getattr(c.weight_broadcast, "timeout", 600.0))
        deadline = time.monotonic() + timeout
        while self.policy.version < c.max_steps - 1:
            if time.monotonic() > deadline:
                self.logger.warning(f"stopping at policy v{self.policy.version}: the trainer did not offer the weights "
                                    f"of step {c.max_steps - 2} within {timeout:.0f}s")
                return
            await asyncio.sleep(0.05)

    async def _metrics_loop(self, max_consecutive_failures: int = 30) -> None:
        """Polls the engines' metrics once a second and feeds the concurrency controller. A scrape
        that fails is logged and retried; after ``max_consecutive_failures`` in a row the task raises,
        which ends the run (the controller would otherwise be silently blind to KV pressure)."""
        failures = 0
        while True:
            await asyncio.sleep(1.0)
            try:
                ms = await self.admin.metrics()
            except asyncio.CancelledError:
                raise
            except Exception as e:
                failures += 1
                self.logger.warning(f"inference metrics scrape failed ({failures}/{max_consecutive_failures}): "
                                    f"{type(e).__name__}: {e}")
                if failures >= max_consecutive_failures:
                    raise RuntimeError("inference metrics endpoint unreachable: concurrency control cannot work "
                                       "(set collect_inference_metrics = false to run without it)") from e
                continue
            failures = 0
            self.inference_metrics.ingest(ms)
            usage = max((m.get("vllm:kv_cache_usage_perc", 0.0) for m in ms), default=0.0)
            waiting = sum(m.get("vllm:num_requests_waiting", 0.0) for m in ms)
            pre = sum(m.get("vllm:num_preemptions_total", 0.0) for m in ms)
            d = self.controller.update(usage, waiting, pre, len(self.dispatcher.inflight))
            if d.cancel:
                self.dispatcher.cancel_newest(d.cancel)

    async def _lag_loop(self, interval: float = 0.25) -> None:
        """Event-loop lag: how late a short sleep wakes up. Long tails mean a coroutine is hogging the loop
        (tokenisation, packing or scoring that should run in a thread) and every request deadline slips
        with it (reference: src/prime_rl/orchestrator/orchestrator.py:394-412)."""
        while True:
            t0 = time.monotonic()
            await asyncio.sleep(interval)
            lag = max(0.0, time.monotonic() - t0 - interval)
            ll = self.loop_lag
            ll["max"], ll["sum"], ll["n"] = max(ll["max"], lag), ll["sum"] + lag, ll["n"] + 1
            if lag > 1.0:
                self.logger.warning(f"event loop was blocked for {lag:.2f}s")

    def _maybe_trigger_eval(self) -> None:
        """Queues one eval epoch per source when the live policy reached a version that is due."""
        ev = self.config.eval
        if ev is None or not self.eval_sources:
            return
        v = self.policy.version
        if v in self._evaluated_versions:
            return
        self._evaluated_versions.add(v)
        if v == 0 and ev.skip_first_step:
            return
        work = []
        for es, src in self.eval_sources:
            interval = es.interval if "interval" in es.model_fields_set else ev.interval
            if v % interval:
                continue
            n = es.num_examples if es.num_examples > 0 else ev.num_examples
            n = min(n if n > 0 else 64, getattr(src.env, "num_tasks", 1 << 30))
            self.eval_sink.expect(src.env.name, v, n, src.group_size)
            work.extend(EvalWork(src, t, v) for t in range(n))
        if work:
            for row in self.eval_sink.abandon(v):           # an older epoch still collecting is superseded
                self._log_eval(row)
            self.dispatcher.request_eval(work)

    def _log_eval(self, row: dict) -> None:
        env, step = row["env"], row["step"]
        self.monitor.log({f"eval/{env}/{k}": v for k, v in row.items() if isinstance(v, (int, float)) and k != "step"},
                         step)
        self.logger.info(f"eval {env} @ policy v{step}: reward {row['reward/mean']:.4f} over {row['rollouts']} rollouts"
                         f" ({row['failed']} failed, {row['cancelled']} cancelled)")
        self.eval_rows.append(row)

    def _handle_lost(self, item: tuple) -> None:
        what, gid, kind, env_name, eval_step, detail = item
        if kind == "eval":
            row = self.eval_sink.fail(env_name, eval_step) if what == "fail" else self.eval_sink.cancel(env_name, eval_step)
            if row is not None:
                self._log_eval(row)
        else:
            self.sink.cancel(gid)
        if what == "fail":
            self.logger.warning(f"{kind} episode failed: {detail}")

    async def run(self) -> None:
        c = self.config
        self.eval_rows: list[dict] = []
        tasks = [asyncio.create_task(self.dispatcher.run()), asyncio.create_task(self.watcher.run()),
                 asyncio.create_task(self._lag_loop())]
        if c.collect_inference_metrics:
            tasks.append(asyncio.create_task(self._metrics_loop()))
        empty = 0
        try:
            while c.max_steps is None or self.step < c.max_steps:
                for t in tasks:
                    if t.done() and t.exception() is not None:
                        raise t.exception()
                self.dispatcher.progress_step = self.step
                self._maybe_trigger_eval()
                try:
                    item = await asyncio.wait_for(self.dispatcher.out_q.get(), timeout=1.0)
                except asyncio.TimeoutError:
                    continue
                if isinstance(item, tuple):
                    self._handle_lost(item)
                    continue
                if item.info.get("_kind") == "eval":
                    row = self.eval_sink.add(item, item.info["_eval_step"])
                    if row is not None:
                        self._log_eval(row)
                    continue
                await self.sink.add(item)
                batch = self.sink.maybe_batch()
                if batch is None:
                    continue
                if not batch:
                    empty += 1
                    if empty >= MAX_EMPTY_BATCHES:
                        raise RuntimeError("aborting: 10 consecutive empty batches")
                    continue
                empty = 0
                m = await self._ship(batch)
                m.update(self.inference_metrics.snapshot())
                ll = self.loop_lag
                m.update({"event_loop_lag/max": ll["max"], "event_loop_lag/mean": ll["sum"] / max(1, ll["n"])})
                ll.update(max=0.0, sum=0.0, n=0)
                self.monitor.log(m, self.step)
                self.logger.info(f"step {self.step} | reward {m['reward']:.3f} | rollouts {m['batch/rollouts']} | "
                                 f"policy v{self.policy.version} | lag {m['off_policy/mean']:.2f}")
                if c.ckpt is not None and c.ckpt.interval and (self.step + 1) % c.ckpt.interval == 0:
                    self.save_ckpt(self.step)
                self.step += 1
            await self._serve_remaining_weight_updates()
        finally:
            # a teardown that hangs (an engine that never answers the aborts, a stuck transport) must not keep
            # the launcher waiting forever: after TEARDOWN_TIMEOUT_S the process ends itself
            watchdog = threading.Timer(TEARDOWN_TIMEOUT_S, lambda: os._exit(1))
            watchdog.daemon = True
            watchdog.start()
            try:
                self.watcher.stopped = True
                await self.dispatcher.stop()
                for t in tasks:
                    t.cancel()
                await asyncio.gather(*tasks, return_exceptions=True)
                self.sender.close()
                await self.client.close()
                await self.admin.close()
                self.monitor.finalize()
            finally:
                watchdog.cancel()


def trace_record(r, step: int) -> dict:
    """What the file monitor keeps of one episode: identity, outcome, and per turn the sampled
    tokens with the engine's log-probabilities (the dashboard's token view reads these)."""
    return {"trace_id": r.trace_id, "step": step, "env": r.env_name, "task_id": r.task_id, "group_id": r.group_id,
            "agent": r.agent, "reward": r.reward, "advantage": r.advantage, "policy_version": r.policy_version,
            "error": r.error, "metrics": r.metrics,
            "turns": [{"prompt_ids": list(t.prompt_ids), "completion_ids": list(t.completion_ids),
                       "completion_logprobs": [round(float(x), 6) for x in t.completion_logprobs],
                       "temperature": t.temperature, "finish_reason": t.finish_reason} for t in r.turns]}


async def run_orchestrator(config: OrchestratorConfig, **kw) -> Orchestrator:
    orch = await Orchestrator(config, **kw).setup()
    await orch.run()
    return orch


def main(argv: list[str] | None = None) -> None:
    from ..configs.base import cli
    from ..utils.logger import setup_logger

    config = cli(OrchestratorConfig, argv)
    if config.dry_run:
        print(config.to_json())
        return
    setup_logger(config.log.level, tag="orchestrator", json_logging=config.log.json_logging)
    try:
        import uvloop

        uvloop.install()
    except ImportError:
        pass
    asyncio.run(run_orchestrator(config))


if __name__ == "__main__":
    main()
