"""Metric sinks. ``setup`` builds the configured monitors; ``log`` fans a metrics row out to
all of them on rank 0 and never raises into the training loop
(reference: src/prime_rl/monitors/__init__.py:42-140)."""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any

from ..utils.logger import get_logger
from ..utils.pathing import get_monitor_dir


class Monitor:
    def log(self, metrics: dict[str, Any], step: int | None) -> None: ...
    def log_trace(self, trace: dict[str, Any]) -> None: ...
    def log_annotations(self, records: list[dict], stream: str) -> None: ...
    def finalize(self) -> None: ...


class FileMonitor(Monitor):
    """``metrics.jsonl`` rows ``{step, time, producer, ...}`` plus chunked trace and
    annotation streams with an index file."""

    def __init__(self, run_dir: Path, producer: str, filename: str = "metrics.jsonl", chunk_size: int = 256):
        self.dir = get_monitor_dir(run_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.path = self.dir / filename
        self.producer = producer
        self.chunk_size = chunk_size
        self._trace_buf: list[dict] = []
        self._trace_chunk = 0
        self._fh = open(self.path, "a", buffering=1)

    def log(self, metrics, step):
        row = {"step": step, "time": time.time(), "producer": self.producer}
        for k, v in metrics.items():
            if hasattr(v, "item"):
                v = v.item()
            row[k] = v
        self._fh.write(json.dumps(row) + "\n")

    def log_trace(self, trace):
        self._trace_buf.append(trace)
        if len(self._trace_buf) >= self.chunk_size:
            self._flush_traces()

    def _flush_traces(self):
        if not self._trace_buf:
            return
        name = f"traces_{self.producer}_{self._trace_chunk:06d}.jsonl"
        with open(self.dir / name, "w") as f:
            for t in self._trace_buf:
                f.write(json.dumps(t) + "\n")
        with open(self.dir / "traces_index.jsonl", "a") as f:
            f.write(json.dumps({"file": name, "count": len(self._trace_buf), "producer": self.producer}) + "\n")
        self._trace_buf = []
        self._trace_chunk += 1

    def log_annotations(self, records, stream):
        with open(self.dir / f"annotations_{stream}.jsonl", "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")

    def finalize(self):
        self._flush_traces()
        self._fh.close()


class WandbMonitor(Monitor):
    def __init__(self, config, run_dir: Path, producer: str, run_config: dict | None = None):
        import os

        import wandb

        mode = "offline" if config.offline else None
        self.run = wandb.init(project=config.project, entity=config.entity, name=config.name, dir=str(run_dir),
                              id=os.environ.get("WANDB_RUN_ID"), resume="allow", mode=mode, config=run_config)
        self.producer = producer

    def log(self, metrics, step):
        self.run.log({k: (v.item() if hasattr(v, "item") else v) for k, v in metrics.items()}, step=step)

    def finalize(self):
        self.run.finish()


class MultiMonitor:
    def __init__(self, monitors: list[Monitor], enabled: bool = True):
        self.monitors, self.enabled = monitors, enabled

    def _each(self, fn_name: str, *args):
        if not self.enabled:
            return
        for m in self.monitors:
            try:
                getattr(m, fn_name)(*args)
            except Exception as e:  # a broken sink must not stop training
                get_logger().warning(f"monitor {type(m).__name__}.{fn_name} failed: {e}")

    def log(self, metrics, step=None):
        self._each("log", metrics, step)

    def log_trace(self, trace):
        self._each("log_trace", trace)

    def log_annotations(self, records, stream="trainer"):
        self._each("log_annotations", records, stream)

    def finalize(self):
        self._each("finalize")


def setup(config, run_dir: Path, producer: str, *, is_master: bool = True, run_config: dict | None = None
          ) -> MultiMonitor:
    mons: list[Monitor] = []
    if is_master and config is not None:
        if config.file is not None:
            fname = str(config.file.path) if config.file.path else "metrics.jsonl"
            mons.append(FileMonitor(run_dir, producer, filename=fname, chunk_size=config.file.trace_chunk_size))
        if config.wandb is not None:
            try:
                mons.append(WandbMonitor(config.wandb, run_dir, producer, run_config))
            except Exception as e:
                get_logger().warning(f"wandb monitor disabled: {e}")
        if getattr(config, "prime", None) is not None:
            from .prime import PrimeMonitor

            mons.append(PrimeMonitor(config.prime, producer, run_config))     # a configured tracker must work: raises
    return MultiMonitor(mons, enabled=is_master)
