"""Run-directory layout.

<run_dir>/configs/attempt_N/resolved/{rl,trainer,orchestrator,inference}.json
<run_dir>/logs/attempt_N/{trainer,orchestrator,inference}.log   (+ ``latest`` symlink)
<run_dir>/checkpoints/step_N/{trainer/,orchestrator/progress.pt}
<run_dir>/broadcasts/step_N/   weights offered to the inference engine (+ marker files)
<run_dir>/batches/step_N/rank_R.bin   packed micro-batches (filesystem transport)
<run_dir>/monitors/file/metrics.jsonl
<run_dir>/weights/step_N/   exported HF checkpoints

Same layout as the reference (src/prime_rl/utils/pathing.py, docs/training.md:326-353).
"""

from __future__ import annotations

import re
import shutil
import time
from pathlib import Path


def get_ckpt_dir(run_dir: Path) -> Path:
    return run_dir / "checkpoints"


def get_step_path(base: Path, step: int) -> Path:
    return base / f"step_{step}"


def get_broadcast_dir(run_dir: Path) -> Path:
    return run_dir / "broadcasts"


def get_batch_dir(run_dir: Path) -> Path:
    return run_dir / "batches"


def get_weights_dir(run_dir: Path) -> Path:
    return run_dir / "weights"


def get_monitor_dir(run_dir: Path) -> Path:
    return run_dir / "monitors" / "file"


def list_steps(base: Path) -> list[int]:
    if not base.exists():
        return []
    out = []
    for p in base.iterdir():
        m = re.fullmatch(r"step_(\d+)", p.name)
        if m and p.is_dir():
            out.append(int(m.group(1)))
    return sorted(out)


def latest_step(base: Path) -> int | None:
    steps = list_steps(base)
    return steps[-1] if steps else None


def next_attempt(run_dir: Path) -> int:
    base = run_dir / "configs"
    if not base.exists():
        return 0
    nums = [int(m.group(1)) for p in base.iterdir() if (m := re.fullmatch(r"attempt_(\d+)", p.name))]
    return max(nums) + 1 if nums else 0


def prepare_attempt_dirs(run_dir: Path) -> tuple[int, Path, Path]:
    """Creates configs/attempt_N/resolved and logs/attempt_N, repoints ``latest``."""
    n = next_attempt(run_dir)
    cfg = run_dir / "configs" / f"attempt_{n}" / "resolved"
    logs = run_dir / "logs" / f"attempt_{n}"
    cfg.mkdir(parents=True, exist_ok=True)
    logs.mkdir(parents=True, exist_ok=True)
    for parent, target in ((run_dir / "logs", logs), (run_dir / "configs", cfg.parent)):
        link = parent / "latest"
        try:
            if link.is_symlink() or link.exists():
                link.unlink()
            link.symlink_to(target.name)
        except OSError:
            pass
    return n, cfg, logs


def clean_future_steps(run_dir: Path, resume_step: int | None) -> None:
    """On resume from step S: drop batches beyond S and broadcasts from S on, so that stale
    artefacts of the abandoned future are never consumed."""
    if resume_step is None:
        return
    for base, keep in ((get_batch_dir(run_dir), lambda s: s <= resume_step),
                       (get_broadcast_dir(run_dir), lambda s: s < resume_step)):
        for s in list_steps(base):
            if not keep(s):
                shutil.rmtree(get_step_path(base, s), ignore_errors=True)


def wait_for_path(path: Path, timeout: float, interval: float = 0.05, what: str = "path") -> None:
    t0 = time.monotonic()
    while not path.exists():
        if time.monotonic() - t0 > timeout:
            raise TimeoutError(f"timed out after {timeout:.0f}s waiting for {what}: {path}")
        time.sleep(interval)
