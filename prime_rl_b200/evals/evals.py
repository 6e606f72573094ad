"""Evals process. Standalone (no ``[online]`` block): every eval source runs once against the weights the
server serves. Online: for every weight step a trainer publishes (``<broadcasts_dir>/step_N`` with its
``.finished`` marker) load the step into the inference server, run each eval source's examples
``group_size`` times, and append one row per (step, env) with mean reward and pass@k to
``<output_dir>/evals.jsonl`` and the monitors. A newer eligible broadcast cancels a running epoch when
``eval.cancel_on_new_checkpoint`` is set
(reference: src/prime_rl/evals/evals.py:1-605, evals/ckpt.py).
"""

from __future__ import annotations

import asyncio
import json
import time
from pathlib import Path
from types import SimpleNamespace

from ..monitors import setup as setup_monitors
from ..orchestrator.clients import AdminPlane, InferenceClient
from ..orchestrator.envs import load_environment
from ..utils.logger import setup_logger

FINISHED = ".finished"      # written by the trainer when a step's weights are complete


def published_steps(watch_dir: Path) -> list[int]:
    """Steps whose weights are complete (marker file present), ascending. ``watch_dir`` is a run directory
    (its ``broadcasts`` folder is read) or the broadcasts folder itself."""
    root = Path(watch_dir)
    if (root / "broadcasts").exists() or root.name != "broadcasts":
        root = root / "broadcasts"
    out = []
    if root.exists():
        for d in root.iterdir():
            if d.name.startswith("step_") and (d / FINISHED).exists():
                try:
                    out.append(int(d.name[5:]))
                except ValueError:
                    pass
    return sorted(out)


def pass_at_k(rewards_per_example: list[list[float]], threshold: float = 1.0) -> float:
    """Fraction of examples with at least one rollout reaching ``threshold``."""
    if not rewards_per_example:
        return 0.0
    return sum(any(r >= threshold for r in rs) for rs in rewards_per_example) / len(rewards_per_example)


def _sampling(cfg, source):
    s = source.sampling if source.sampling.temperature is not None or source.sampling.max_completion_tokens else cfg.sampling
    return SimpleNamespace(temperature=s.temperature if s.temperature is not None else 0.0,
                           top_p=s.top_p if s.top_p is not None else 1.0, top_k=s.top_k,
                           max_completion_tokens=s.max_completion_tokens, extra_body=s.extra_body)


async def evaluate_once(config, client, step: int, sem: asyncio.Semaphore, skip=()) -> list[dict]:
    rows = []
    for source in config.eval.source:
        if source.resolved_name in skip:
            continue
        env = load_environment(source)
        sampling = _sampling(config.eval, source)
        n = source.num_examples if source.num_examples > 0 else (config.eval.num_examples if config.eval.num_examples > 0 else 64)
        n = min(n, env.num_tasks)
        g = max(source.group_size, config.eval.group_size)

        async def one(task_id: int, j: int):
            async with sem:
                task = env.task(task_id)
                sampling_j = SimpleNamespace(**{**vars(sampling), "max_completion_tokens":
                                                sampling.max_completion_tokens or task.get("max_tokens")})
                r = await env.rollout(client, task_id, sampling_j, step, f"eval-{task_id}")
                return task_id, r.reward, sum(len(t.completion_ids) for t in r.turns)

        t0 = time.monotonic()
        results = await asyncio.gather(*[one(t, j) for t in range(n) for j in range(g)])
        per_example: dict[int, list[float]] = {}
        for tid, rew, _ in results:
            per_example.setdefault(tid, []).append(rew)
        rewards = [r for _, r, _ in results]
        rows.append({"step": step, "env": env.name, "num_examples": n, "group_size": g,
                     "reward/mean": sum(rewards) / max(len(rewards), 1),
                     f"pass@{g}": pass_at_k(list(per_example.values())),
                     "completion_len/mean": sum(c for _, _, c in results) / max(len(results), 1),
                     "time": time.monotonic() - t0})
    return rows


async def run_evals(config) -> list[dict]:
    log = setup_logger(config.log.level or "info", tag="evals")
    out_dir = Path(config.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    monitor = setup_monitors(config.monitors, out_dir, producer="evals")
    ev = config.eval
    client = InferenceClient(ev.client, config.model)
    admin = AdminPlane(ev.client)
    band = ev.concurrency
    sem = asyncio.Semaphore(band.initial_inflight or band.max_inflight or 256)
    online = config.online
    done: set[int] = set()
    all_rows: list[dict] = []
    results = out_dir / "evals.jsonl"
    progress = out_dir / "evals_progress.json"
    if config.resume is not None and progress.exists():            # standalone resume: skip finished sources
        done_envs = set(json.loads(progress.read_text()).get("envs", []))
    else:
        done_envs = set()

    async def run_step(step: int, load: bool):
        if load:
            await admin.pause()
            try:
                await admin.update_weights(str(Path(online.broadcasts_dir) / f"step_{step}"))
            finally:
                await admin.resume()
        rows = await evaluate_once(config, client, step, sem, skip=done_envs)
        with open(results, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
                monitor.log({f"eval/{r['env']}/{k}": v for k, v in r.items() if isinstance(v, (int, float))}, step=step)
                log.info(f"step {step} {r['env']}: reward {r['reward/mean']:.4f}")
                if config.ckpt is not None:
                    done_envs.add(r["env"])
                    progress.write_text(json.dumps({"envs": sorted(done_envs)}))
        all_rows.extend(rows)

    def eligible() -> list[int]:
        first = (online.resume_step or -1)
        steps = [s for s in published_steps(online.broadcasts_dir) if s not in done and s > first
                 and s % ev.interval == 0]
        if ev.skip_first_step:
            steps = [s for s in steps if s != 0]
        return steps

    try:
        if online is None:
            await run_step(0, load=False)
            return all_rows
        if ev.retrigger_on_resume and online.resume_step is not None and online.resume_step % ev.interval == 0:
            await run_step(online.resume_step, load=True)
        while True:
            for s in eligible():
                task = asyncio.create_task(run_step(s, load=True))
                while not task.done():
                    await asyncio.sleep(min(online.poll_interval, 0.5))
                    if ev.cancel_on_new_checkpoint and any(n > s for n in eligible()):
                        task.cancel()              # newer weights are waiting: this epoch is stale
                        log.info(f"eval epoch of step {s} cancelled: a newer broadcast is ready")
                        break
                try:
                    await task
                except asyncio.CancelledError:
                    pass
                done.add(s)
            if online.max_steps is not None and done and max(done) >= online.max_steps:
                return all_rows
            await asyncio.sleep(online.poll_interval)
    finally:
        await client.close()
        monitor.finalize()
        await admin.close()
