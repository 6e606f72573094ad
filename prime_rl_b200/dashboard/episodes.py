"""Episode store of the dashboard: an incrementally maintained index over the file monitor's trace chunks with
the queries the trace browser needs (filtered / sorted pages, histograms, per-step series, rollout groups of
one task, per-episode timelines merged with the trainer's annotations), metric down-sampling and paged log reads.

Same views as the reference's dashboard backend (src/prime_rl/dashboard/server.py:1496-1985: ``/episodes``,
``/episodes/histogram``, ``/episodes/series``, ``/rollouts``, ``/episodes/{line}/timeline``, ``/log``), over this
package's own trace format (``orchestrator/orchestrator.py: trace_record``).
"""

from __future__ import annotations

import json
import math
import threading
from pathlib import Path

SUMMARY_FIELDS = ("reward", "advantage", "tokens", "turns", "step", "policy_version", "prompt_tokens", "lag")


def summarise(t: dict, file: str, line: int) -> dict:
    turns = t.get("turns", [])
    comp = sum(len(u.get("completion_ids", [])) for u in turns)
    prompt = len(turns[0].get("prompt_ids", [])) if turns else 0
    lp = [x for u in turns for x in u.get("completion_logprobs", [])]
    step, ver = t.get("step"), t.get("policy_version")
    return {"trace_id": t.get("trace_id"), "step": step, "env": t.get("env"), "task_id": t.get("task_id"),
            "group_id": t.get("group_id"), "agent": t.get("agent"), "reward": t.get("reward"),
            "advantage": t.get("advantage"), "policy_version": ver, "error": t.get("error"),
            "turns": len(turns), "tokens": comp, "prompt_tokens": prompt,
            "mean_logprob": (sum(lp) / len(lp)) if lp else None,
            "lag": (step - 1 - ver) if isinstance(step, int) and isinstance(ver, int) else None,
            "finish_reason": turns[-1].get("finish_reason") if turns else None, "file": file, "line": line}


class EpisodeIndex:
    """Summaries of all episodes of one run. Chunk files are append-only and never rewritten, so a refresh reads
    only files it has not seen (and re-reads the newest one when it grew)."""

    def __init__(self, monitor_dir: Path):
        self.dir = Path(monitor_dir)
        self.rows: list[dict] = []
        self._seen: dict[str, tuple[int, int]] = {}       # file -> (size, rows taken from it)
        self._lock = threading.Lock()

    def refresh(self) -> "EpisodeIndex":
        with self._lock:
            for f in sorted(self.dir.glob("traces_*_*.jsonl")):
                try:
                    size = f.stat().st_size
                except OSError:
                    continue
                old_size, taken = self._seen.get(f.name, (0, 0))
                if size == old_size:
                    continue
                try:
                    with open(f) as fh:
                        for line_no, line in enumerate(fh):
                            if line_no < taken:
                                continue
                            try:
                                t = json.loads(line)
                            except ValueError:
                                break                      # a row that is still being written: next refresh
                            self.rows.append(summarise(t, f.name, line_no))
                            taken = line_no + 1
                except OSError:
                    continue
                self._seen[f.name] = (size, taken)
        return self

    # ------------------------------------------------------------------ queries
    def select(self, *, step: int | None = None, min_step: int | None = None, max_step: int | None = None,
               env: str | None = None, task_id=None, group_id: str | None = None, min_reward: float | None = None,
               max_reward: float | None = None, errors: bool | None = None, text: str | None = None) -> list[dict]:
        out = []
        for r in self.rows:
            if step is not None and r["step"] != step:
                continue
            if min_step is not None and (r["step"] is None or r["step"] < min_step):
                continue
            if max_step is not None and (r["step"] is None or r["step"] > max_step):
                continue
            if env is not None and r["env"] != env:
                continue
            if task_id is not None and str(r["task_id"]) != str(task_id):
                continue
            if group_id is not None and r["group_id"] != group_id:
                continue
            if min_reward is not None and (r["reward"] is None or r["reward"] < min_reward):
                continue
            if max_reward is not None and (r["reward"] is None or r["reward"] > max_reward):
                continue
            if errors is not None and bool(r["error"]) != errors:
                continue
            if text and text not in str(r["trace_id"]) and text not in str(r["env"]) and text not in str(r["error"]):
                continue
            out.append(r)
        return out

    def page(self, rows: list[dict], *, sort: str = "step", descending: bool = True, offset: int = 0,
             limit: int = 100) -> dict:
        key = sort if sort in SUMMARY_FIELDS or sort in ("env", "trace_id", "mean_logprob") else "step"
        none_last = [r for r in rows if r.get(key) is None]
        some = sorted((r for r in rows if r.get(key) is not None), key=lambda r: r[key], reverse=descending)
        ordered = some + none_last
        return {"total": len(ordered), "offset": offset, "rows": ordered[offset:offset + max(0, min(limit, 1000))],
                "envs": sorted({r["env"] for r in self.rows if r["env"] is not None}),
                "steps": [min((r["step"] for r in self.rows if r["step"] is not None), default=None),
                          max((r["step"] for r in self.rows if r["step"] is not None), default=None)]}

    @staticmethod
    def histogram(rows: list[dict], field: str = "reward", bins: int = 20) -> dict:
        vals = [r[field] for r in rows if isinstance(r.get(field), (int, float)) and math.isfinite(r[field])]
        if not vals:
            return {"field": field, "edges": [], "counts": [], "n": 0}
        lo, hi = min(vals), max(vals)
        if hi == lo:
            return {"field": field, "edges": [lo, hi], "counts": [len(vals)], "n": len(vals), "mean": lo}
        bins = max(1, min(bins, 200))
        counts = [0] * bins
        w = (hi - lo) / bins
        for v in vals:
            counts[min(bins - 1, int((v - lo) / w))] += 1
        return {"field": field, "edges": [lo + i * w for i in range(bins + 1)], "counts": counts, "n": len(vals),
                "mean": sum(vals) / len(vals)}

    @staticmethod
    def series(rows: list[dict], field: str = "reward") -> list[dict]:
        """Per step: count, mean, min, max, and the quartiles of ``field``."""
        by_step: dict[int, list[float]] = {}
        for r in rows:
            v = r.get(field)
            if r["step"] is not None and isinstance(v, (int, float)) and math.isfinite(v):
                by_step.setdefault(r["step"], []).append(v)
        out = []
        for s in sorted(by_step):
            v = sorted(by_step[s])
            q = lambda p: v[min(len(v) - 1, int(p * (len(v) - 1) + 0.5))]   # noqa: E731
            out.append({"step": s, "count": len(v), "mean": sum(v) / len(v), "min": v[0], "max": v[-1],
                        "p25": q(0.25), "p50": q(0.5), "p75": q(0.75)})
        return out

    @staticmethod
    def rollouts(rows: list[dict]) -> list[dict]:
        """The samples of one task side by side: one entry per ``group_id`` with its members' rewards."""
        groups: dict[str, dict] = {}
        for r in rows:
            g = groups.setdefault(str(r["group_id"]), {"group_id": r["group_id"], "env": r["env"], "task_id": r["task_id"],
                                                        "step": r["step"], "members": []})
            g["members"].append({k: r[k] for k in ("trace_id", "reward", "advantage", "tokens", "error",
                                                   "finish_reason", "policy_version")})
        out = []
        for g in groups.values():
            rew = [m["reward"] for m in g["members"] if isinstance(m["reward"], (int, float))]
            g["size"] = len(g["members"])
            g["reward_mean"] = sum(rew) / len(rew) if rew else None
            g["reward_spread"] = (max(rew) - min(rew)) if rew else None
            g["solved"] = sum(1 for x in rew if x > 0)
            out.append(g)
        out.sort(key=lambda g: (g["step"] is None, g["step"]), reverse=True)
        return out


def timeline(trace: dict) -> list[dict]:
    """Turn-by-turn account of one episode (``dashboard.server.read_trace`` output): token counts, the engine's
    summed log-probability, and where the trainer annotated the branch, its own sum, the mean absolute
    per-token gap, mean entropy and the number of tokens that took part in the loss."""
    ann = {a.get("branch_index", i): a for i, a in enumerate(trace.get("annotations", []))}
    out = []
    turns = trace.get("turns", [])
    for i, t in enumerate(turns):
        lp = [float(x) for x in t.get("completion_logprobs", [])]
        row = {"turn": i, "prompt_tokens": len(t.get("prompt_ids", [])), "completion_tokens": len(lp),
               "engine_logprob_sum": sum(lp), "finish_reason": t.get("finish_reason"),
               "temperature": t.get("temperature")}
        a = ann.get(i) or (ann.get(-1) if i == len(turns) - 1 else None) or \
            (next(iter(ann.values())) if (len(ann) == 1 and i == len(turns) - 1) else None)
        if a is not None and lp:
            off = row["prompt_tokens"]
            tl = [float(x) for x in a.get("logprobs", [])[off:off + len(lp)]]
            if len(tl) == len(lp):
                ent = [float(x) for x in a.get("entropy", [])[off:off + len(lp)]]
                mask = a.get("loss_mask", [])[off:off + len(lp)]
                row.update(trainer_logprob_sum=sum(tl),
                           mean_abs_gap=sum(abs(x - y) for x, y in zip(tl, lp)) / len(lp),
                           mismatch_kl=sum(math.exp(y - x) - (y - x) - 1 for x, y in zip(tl, lp)) / len(lp),
                           mean_entropy=(sum(ent) / len(ent)) if ent else None,
                           loss_tokens=sum(1 for m in mask if m))
        out.append(row)
    return out


def downsample(rows: list[dict], key: str, points: int = 2000, producer: str | None = None) -> list[dict]:
    """(step, value) pairs of one metric, averaged into at most ``points`` buckets over the step range."""
    pts = [(r["step"], r[key]) for r in rows
           if isinstance(r.get("step"), int) and isinstance(r.get(key), (int, float)) and math.isfinite(r[key])
           and (producer is None or r.get("producer") == producer)]
    if len(pts) <= points:
        return [{"step": s, "value": v} for s, v in pts]
    lo, hi = min(s for s, _ in pts), max(s for s, _ in pts)
    w = max(1, math.ceil((hi - lo + 1) / points))
    acc: dict[int, list[float]] = {}
    for s, v in pts:
        acc.setdefault((s - lo) // w, []).append(v)
    return [{"step": lo + b * w, "value": sum(v) / len(v), "min": min(v), "max": max(v), "count": len(v)}
            for b, v in sorted(acc.items())]


def read_log(run_dir: Path, name: str, offset: int | None = None, lines: int = 400) -> dict:
    """``lines`` lines of a log file of the run starting at byte ``offset`` (None = the tail). Returns the text,
    the byte range and the file size, so that a viewer can page backwards and follow the end."""
    root = Path(run_dir).resolve()
    path = (root / name).resolve()
    if root not in path.parents or path.suffix not in (".log", ".out", ".err", ".txt", ".jsonl"):
        raise PermissionError("not a log file of this run")
    size = path.stat().st_size
    with open(path, "rb") as fh:
        if offset is None:
            start = max(0, size - 256 * 1024)
            fh.seek(start)
            data = fh.read()
            cut = data.split(b"\n")
            if start > 0:
                cut = cut[1:]
            tail = cut[-lines:] if lines > 0 else cut
            text = b"\n".join(tail)
            begin = size - len(text)
            return {"name": name, "start": begin, "end": size, "size": size, "text": text.decode(errors="replace")}
        fh.seek(max(0, min(offset, size)))
        data = fh.read(1 << 20)
        cut = data.split(b"\n")[:lines]
        text = b"\n".join(cut)
        return {"name": name, "start": offset, "end": offset + len(text) + (1 if len(cut) == lines else 0),
                "size": size, "text": text.decode(errors="replace")}
