"""Rolling view of the engines' Prometheus-style metrics for the orchestrator's own logs.

Every scrape (one dict per engine, names as the engines export them: ``vllm:kv_cache_usage_perc``,
``vllm:num_requests_running`` / ``_waiting``, ``vllm:generation_tokens_total``, ``vllm:prompt_tokens_total``,
``vllm:num_preemptions_total``, ``vllm:prefix_cache_hits_total`` / ``_queries_total``) is folded into gauges,
counter rates and a histogram of KV usage over the window since the last ``snapshot()``; the snapshot goes
out with the step metrics under ``inference/``. With prefill / decode roles the engines can be told apart by
a ``role`` label. Same job as the reference's collector (src/prime_rl/orchestrator/inference_metrics.py:36-458).
"""

from __future__ import annotations

import time

_KV_EDGES = (0.1, 0.25, 0.5, 0.6, 0.7, 0.8, 0.9, 0.95, 1.01)
_COUNTERS = {"vllm:generation_tokens_total": "generation_tokens", "vllm:prompt_tokens_total": "prompt_tokens",
             "vllm:num_preemptions_total": "preemptions", "vllm:prefix_cache_hits_total": "prefix_hits",
             "vllm:prefix_cache_queries_total": "prefix_queries", "vllm:request_success_total": "requests_finished"}
_GAUGES = {"vllm:kv_cache_usage_perc": "kv_usage", "vllm:num_requests_running": "running",
           "vllm:num_requests_waiting": "waiting"}


class InferenceMetrics:
    def __init__(self, roles: list[str] | None = None):
        self.roles = roles
        self._reset_window()
        self._last_counters: dict[tuple[int, str], float] = {}
        self._window_counters: dict[str, float] = {}
        self._t0 = time.monotonic()

    def _reset_window(self) -> None:
        self._gauge_sum: dict[str, float] = {}
        self._gauge_max: dict[str, float] = {}
        self._gauge_n = 0
        self._kv_hist = [0] * len(_KV_EDGES)
        self._window_counters = {}
        self._t0 = time.monotonic()

    def ingest(self, per_engine: list[dict]) -> None:
        """One scrape: a metrics dict per engine (in a stable engine order)."""
        for idx, m in enumerate(per_engine):
            role = m.get("role")
            if self.roles is not None and role is not None and role not in self.roles:
                continue
            for src, name in _GAUGES.items():
                v = float(m.get(src, 0.0))
                self._gauge_sum[name] = self._gauge_sum.get(name, 0.0) + v
                self._gauge_max[name] = max(self._gauge_max.get(name, 0.0), v)
            self._gauge_n += 1
            kv = float(m.get("vllm:kv_cache_usage_perc", 0.0))
            for b, edge in enumerate(_KV_EDGES):
                if kv < edge:
                    self._kv_hist[b] += 1
                    break
            for src, name in _COUNTERS.items():
                if src not in m:
                    continue
                v = float(m[src])
                last = self._last_counters.get((idx, src))
                if last is not None and v >= last:           # a restarted engine starts from zero again
                    self._window_counters[name] = self._window_counters.get(name, 0.0) + (v - last)
                self._last_counters[(idx, src)] = v

    def snapshot(self) -> dict[str, float]:
        """Metrics of the window since the previous snapshot (and starts a new window)."""
        dt = max(time.monotonic() - self._t0, 1e-6)
        out: dict[str, float] = {}
        n = max(1, self._gauge_n)
        for name, total in self._gauge_sum.items():
            out[f"inference/{name}/mean"] = total / n
            out[f"inference/{name}/max"] = self._gauge_max[name]
        for name, delta in self._window_counters.items():
            out[f"inference/{name}/per_s"] = delta / dt
        q = self._window_counters.get("prefix_queries", 0.0)
        if q > 0:
            out["inference/prefix_hit_rate"] = self._window_counters.get("prefix_hits", 0.0) / q
        total = sum(self._kv_hist)
        if total:
            lo = 0.0
            for count, edge in zip(self._kv_hist, _KV_EDGES):
                out[f"inference/kv_usage_hist/{lo:.2f}-{min(edge, 1.0):.2f}"] = count / total
                lo = edge
        out["inference/scrapes"] = float(self._gauge_n)
        self._reset_window()
        return out
