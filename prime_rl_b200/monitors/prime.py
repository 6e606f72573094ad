"""Platform monitor: ships metrics and sampled episodes of a run to a hosted run tracker over HTTP.

Same role as the reference's ``PrimeMonitor`` (src/prime_rl/monitors/prime.py:31-116), which delegates to an
SDK that is not part of this package. Here the protocol is spelled out and owned by this file:

* ``POST {base}/runs``                       register a run (name, model, environments, training spec, config)
  -> ``{"id": ..., "url": ...}``; skipped when ``$RUN_ID`` names a run that a managed launch created (attach);
* ``POST {base}/runs/{id}/metrics``          one row ``{"step", "timestamp", "metrics"}`` per logged step;
* ``POST {base}/runs/{id}/samples``          every ``sample_every``-th step: the step's traces as one Parquet
  file (pyarrow; JSON lines when pyarrow is missing), multipart-free: body = file bytes, step in the query;
* ``POST {base}/runs/{id}/status``           ``completed`` from ``finalize``, ``crashed`` from the exit hook of a
  process that ends without finalizing (not for attached runs: their launcher owns the failure marking).

All network I/O happens on one uploader thread fed by a bounded queue: logging never blocks the training or
orchestration loop for longer than a queue put, failed requests are retried with back-off, and when the queue
is full the oldest *metrics* rows are dropped first (status changes never are). ``finalize`` drains the queue
for at most ``finish_timeout`` seconds. ``$PRIME_RUNS_MODE=disabled`` turns the monitor into a no-op; a
configured monitor without an API key raises at start-up rather than training untracked.
"""

from __future__ import annotations

import atexit
import io
import json
import math
import os
import queue
import threading
import time
from typing import Any

from ..utils.logger import get_logger
from . import Monitor

BASE_URL_VAR = "PRIME_API_BASE"
MODE_VAR = "PRIME_RUNS_MODE"
FINISH_TIMEOUT = 60.0


def resolve_base_url(configured: str) -> str:
    """``$PRIME_API_BASE`` historically points at the fine-tuning API root (``.../api/v1/rft``); the run tracker
    lives beside it, so that suffix is dropped."""
    base = os.getenv(BASE_URL_VAR) or configured
    return base.rstrip("/").removesuffix("/rft")


def sanitize(metrics: dict[str, Any]) -> tuple[dict[str, Any], list[str]]:
    """Numbers only, finite only; returns the clean row and the names that were dropped."""
    clean, dropped = {}, []
    for k, v in metrics.items():
        if hasattr(v, "item"):
            v = v.item()
        if isinstance(v, bool):
            clean[k] = int(v)
        elif isinstance(v, (int, float)):
            if math.isfinite(v):
                clean[k] = v
            else:
                dropped.append(k)
        elif isinstance(v, str):
            clean[k] = v
        else:
            dropped.append(k)
    return clean, dropped


def encode_samples(traces: list[dict]) -> tuple[bytes, str]:
    """Traces of one step as a Parquet table (nested fields as JSON strings) or JSON lines."""
    flat = [{k: (v if isinstance(v, (int, float, str, bool)) or v is None else json.dumps(v)) for k, v in t.items()}
            for t in traces]
    try:
        import pyarrow as pa
        import pyarrow.parquet as pq

        keys = sorted({k for r in flat for k in r})
        table = pa.table({k: [r.get(k) for r in flat] for k in keys})
        buf = io.BytesIO()
        pq.write_table(table, buf, compression="zstd")
        return buf.getvalue(), "application/vnd.apache.parquet"
    except Exception:
        return "\n".join(json.dumps(r) for r in flat).encode(), "application/x-ndjson"


class PrimeMonitor(Monitor):
    def __init__(self, config, producer: str, run_config: dict | None = None, *, client=None,
                 sample_every: int = 10, queue_size: int = 512, finish_timeout: float = FINISH_TIMEOUT,
                 max_retries: int = 5):
        self.log_ = get_logger()
        self.producer, self.sample_every, self.finish_timeout, self.max_retries = producer, sample_every, \
            finish_timeout, max_retries
        self.enabled = os.getenv(MODE_VAR, "online") != "disabled"
        self.run_id: str | None = None
        self.url: str | None = None
        self.attached = False
        self.dropped_rows = 0
        self._finalized = False
        self._traces: list[dict] = []
        self._trace_step: int | None = None
        self._q: queue.Queue = queue.Queue(maxsize=queue_size)
        if not self.enabled:
            self.log_.info(f"platform monitor disabled ({MODE_VAR}=disabled)")
            return
        key = os.getenv(config.api_key_var)
        if client is None:
            if not key:
                raise RuntimeError(f"the platform monitor is configured but ${config.api_key_var} is not set "
                                   f"(set {MODE_VAR}=disabled to train untracked)")
            import httpx

            client = httpx.Client(base_url=resolve_base_url(config.base_url), timeout=30.0,
                                  headers={"Authorization": f"Bearer {key}"})
        self.client = client
        if run_id := os.getenv("RUN_ID"):
            self.run_id, self.attached = run_id, True          # a managed launch created the run: attach
        else:
            rc = run_config or {}
            body = {"name": config.run_name or rc.get("run", {}).get("name") or producer, "kind": "train",
                    "model": (rc.get("model") or {}).get("name", "unknown") if isinstance(rc.get("model"), dict)
                    else (rc.get("model") or "unknown"),
                    "environments": [s.get("id") or s.get("name") for s in (rc.get("train") or {}).get("source", [])
                                     if isinstance(s, dict)],
                    "training": {k: rc.get(k) for k in ("max_steps", "batch_size", "group_size", "seq_len")
                                 if rc.get(k) is not None},
                    "config": rc}
            r = self.client.post("/runs", json=body)
            r.raise_for_status()
            data = r.json()
            self.run_id, self.url = str(data["id"]), data.get("url")
        self.log_.info(f"logging metrics and episodes to platform run {self.run_id}"
                       + (" (attached via $RUN_ID)" if self.attached else "") + (f" ({self.url})" if self.url else ""))
        self._worker = threading.Thread(target=self._drain, name="prime-monitor", daemon=True)
        self._worker.start()
        atexit.register(self._at_exit)

    # ------------------------------------------------------------------ producer side
    def _put(self, item: tuple, droppable: bool) -> None:
        while True:
            try:
                self._q.put_nowait(item)
                return
            except queue.Full:
                if droppable:
                    self.dropped_rows += 1                    # back-pressure: this row is lost, the loop goes on
                    return
                try:                                          # make room for a status change
                    self._q.get_nowait()
                    self._q.task_done()
                    self.dropped_rows += 1
                except queue.Empty:
                    pass

    def log(self, metrics, step):
        if not self.enabled or self._finalized:
            return
        clean, dropped = sanitize(metrics)
        if dropped:
            self.log_.warning(f"dropping {len(dropped)} non-numeric or non-finite metric value(s): "
                              + ", ".join(dropped[:5]))
        self._put(("metrics", {"step": step, "timestamp": time.time(), "producer": self.producer,
                               "metrics": clean}), True)

    def log_trace(self, trace):
        """Traces are grouped by their step; a step that falls on the sampling cadence is uploaded when the next
        step's first trace (or ``finalize``) shows that it is complete."""
        if not self.enabled or self._finalized:
            return
        step = trace.get("step")
        if self._trace_step is not None and step != self._trace_step:
            self._flush_traces()
        self._trace_step = step
        if step is not None and step % self.sample_every == 0:
            self._traces.append(trace)

    def _flush_traces(self):
        if self._traces:
            body, ctype = encode_samples(self._traces)
            self._put(("samples", (self._trace_step, body, ctype, len(self._traces))), True)
        self._traces = []

    def finalize(self, status: str = "completed"):
        if not self.enabled or self._finalized:
            return
        self._flush_traces()
        self._finalized = True
        if not (self.attached and status != "completed"):
            self._put(("status", {"status": status, "dropped_rows": self.dropped_rows}), False)
        self._put(("stop", None), False)
        self._worker.join(self.finish_timeout)
        if self._worker.is_alive():
            self.log_.warning(f"platform monitor: uploads still queued after {self.finish_timeout}s, giving up")

    def _at_exit(self):
        if self.enabled and not self._finalized:
            self.finalize("crashed")

    # ------------------------------------------------------------------ uploader thread
    def _send(self, kind: str, payload) -> None:
        base = f"/runs/{self.run_id}"
        if kind == "metrics":
            r = self.client.post(base + "/metrics", json=payload)
        elif kind == "status":
            r = self.client.post(base + "/status", json=payload)
        else:
            step, body, ctype, n = payload
            r = self.client.post(base + "/samples", params={"step": step, "count": n}, content=body,
                                 headers={"Content-Type": ctype})
        if r.status_code >= 500 or r.status_code == 429:
            raise ConnectionError(f"{kind}: HTTP {r.status_code}")
        if r.status_code >= 400:                              # a request the server rejects will not get better
            self.log_.warning(f"platform monitor: {kind} rejected with HTTP {r.status_code}")

    def _drain(self):
        while True:
            kind, payload = self._q.get()
            try:
                if kind == "stop":
                    return
                delay = 0.5
                for attempt in range(self.max_retries):
                    try:
                        self._send(kind, payload)
                        break
                    except Exception as e:                    # network errors, 5xx, 429: retry with back-off
                        if attempt == self.max_retries - 1:
                            self.log_.warning(f"platform monitor: giving up on a {kind} upload: {e}")
                        else:
                            time.sleep(delay)
                            delay = min(delay * 2, 8.0)
            finally:
                self._q.task_done()
