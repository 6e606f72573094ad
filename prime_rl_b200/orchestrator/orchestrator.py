"""Asynchronous RL orchestrator: schedules environment episodes against the inference pool,
scores completed groups, packs samples into per-rank micro-batches for the trainer and
relays new policy versions into the engines.

Asynchrony contract (reference: src/prime_rl/orchestrator/orchestrator.py:95-98, :634-652):
batch ``step`` is shipped only once the engines run policy version >= ``step - 1 -
TARGET_LAG``; rollouts generated more than ``max_off_policy_steps`` versions ago are dropped.

Parts:
  Dispatcher     keeps up to the controller's limit of episodes in flight, one group per task
  TrainSink      groups -> advantages -> samples -> pending batch (stale / zero-advantage pruning)
  WeightWatcher  polls ``broadcasts/`` for offered versions and runs the receiver handshake
  Orchestrator   main loop, metrics, checkpoints
"""

from __future__ import annotations

import asyncio
import random
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
from .types import Policy, Rollout

TARGET_LAG = 1
MAX_EMPTY_BATCHES = 10


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
    """Fills the in-flight budget with group episodes; finished rollouts go to ``out_q``."""

    def __init__(self, sources: list[Source], client: InferenceClient, policy: Policy,
                 controller: ConcurrencyController, seed: int = 0, tasks_per_minute: int | None = None):
        self.sources, self.client, self.policy, self.controller = sources, client, policy, controller
        self.out_q: asyncio.Queue = asyncio.Queue()
        self.inflight: dict[asyncio.Task, str] = {}
        self.rng = random.Random(seed)
        self.paused = asyncio.Event()
        self.paused.set()
        self.stopped = False
        self.min_fresh_version = 0
        self.tasks_per_minute = tasks_per_minute
        self._last_launch = 0.0
        self.stats = defaultdict(int)

    def _pick(self) -> Source:
        total = sum(s.ratio for s in self.sources)
        x = self.rng.random() * total
        for s in self.sources:
            x -= s.ratio
            if x <= 0:
                return s
        return self.sources[-1]

    async def _episode(self, src: Source, task_id: int, group_id: str) -> None:
        version = self.policy.version
        try:
            r: Rollout = await src.env.rollout(self.client, task_id, src.sampling, version, group_id)
            await src.algo.finalize_episode(r)
            r.info["_source"] = src
            await self.out_q.put(r)
            self.stats["episodes_ok"] += 1
        except asyncio.CancelledError:
            self.stats["episodes_cancelled"] += 1
            await self.out_q.put(("cancel", group_id))
            raise
        except Exception as e:
            self.stats["episodes_failed"] += 1
            await self.out_q.put(("fail", group_id, repr(e)))
        finally:
            self.controller.on_episode_done()

    def _launch_group(self) -> None:
        src = self._pick()
        if src.sampler is not None:
            task_id = src.sampler.sample()
            src.next_task = getattr(src.sampler, "next", src.next_task)
        else:
            task_id = src.next_task % max(1, getattr(src.env, "num_tasks", 1 << 30))
            src.next_task += 1
        gid = uuid.uuid4().hex
        for _ in range(src.group_size):
            t = asyncio.create_task(self._episode(src, task_id, gid))
            self.inflight[t] = gid
            t.add_done_callback(lambda t: self.inflight.pop(t, None))
        self.stats["groups_launched"] += 1

    async def run(self) -> None:
        while not self.stopped:
            await self.paused.wait()
            room = self.controller.limit - len(self.inflight)
            gs = min(s.group_size for s in self.sources)
            if room >= gs:
                if self.tasks_per_minute:
                    wait = 60.0 / self.tasks_per_minute - (time.monotonic() - self._last_launch)
                    if wait > 0:
                        await asyncio.sleep(wait)
                self._launch_group()
                self._last_launch = time.monotonic()
                await asyncio.sleep(0)
            else:
                await asyncio.sleep(0.005)

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
        self.zero_output_batches = 0

    def cancel(self, group_id: str) -> None:
        self.groups.pop(group_id, None)
        self.dead_groups.add(group_id)

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
            return
        await src.algo.score_group(group)
        if src.sampler is not None:
            src.sampler.update(group[0].task_id, sum(r.reward for r in group) / len(group))
        advs = [r.advantage or 0.0 for r in group]
        for gate in src.gates:
            if all(gate.reject_min <= a <= gate.reject_max for a in advs):
                self.stats["groups_rejected_by_gate"] += 1
                return
        self.stats["groups_scored"] += 1
        for r in group:
            self.stats["reward_sum"] += r.reward
            self.stats["reward_n"] += 1
            if src.algo.action_loss_type == "rl" and (r.advantage or 0.0) == 0.0 \
                    and src.algo.observation_weights(r, 0) is None:
                self.stats["rollouts_pruned_zero_adv"] += 1
                continue     # contributes no gradient
            self.pending.append((r, src.algo.to_samples(r)))

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
        await self.receiver.receive(step)
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
                                     tasks_per_minute=c.tasks_per_minute)
        self.sink = TrainSink(c, self.policy)
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
            usage = max((m.get("vllm:kv_cache_usage_perc", 0.0) for m in ms), default=0.0)
            waiting = sum(m.get("vllm:num_requests_waiting", 0.0) for m in ms)
            pre = sum(m.get("vllm:num_preemptions_total", 0.0) for m in ms)
            d = self.controller.update(usage, waiting, pre, len(self.dispatcher.inflight))
            if d.cancel:
                self.dispatcher.cancel_newest(d.cancel)

    async def run(self) -> None:
        c = self.config
        tasks = [asyncio.create_task(self.dispatcher.run()), asyncio.create_task(self.watcher.run())]
        if c.collect_inference_metrics:
            tasks.append(asyncio.create_task(self._metrics_loop()))
        empty = 0
        try:
            while c.max_steps is None or self.step < c.max_steps:
                for t in tasks:
                    if t.done() and t.exception() is not None:
                        raise t.exception()
                try:
                    item = await asyncio.wait_for(self.dispatcher.out_q.get(), timeout=1.0)
                except asyncio.TimeoutError:
                    continue
                if isinstance(item, tuple):
                    self.sink.cancel(item[1])
                    if item[0] == "fail":
                        self.logger.warning(f"episode failed: {item[2]}")
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
                self.monitor.log(m, self.step)
                self.logger.info(f"step {self.step} | reward {m['reward']:.3f} | rollouts {m['batch/rollouts']} | "
                                 f"policy v{self.policy.version} | lag {m['off_policy/mean']:.2f}")
                if c.ckpt is not None and c.ckpt.interval and (self.step + 1) % c.ckpt.interval == 0:
                    self.save_ckpt(self.step)
                self.step += 1
        finally:
            self.watcher.stopped = True
            await self.dispatcher.stop()
            for t in tasks:
                t.cancel()
            await asyncio.gather(*tasks, return_exceptions=True)
            self.sender.close()
            await self.client.close()
            await self.admin.close()
            self.monitor.finalize()


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
