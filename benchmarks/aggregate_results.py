"""Collects benchmark result files (this framework's ``run_single_benchmark.py`` and the
reference's ``benchmarks/baselines/*.json`` share one layout) into a markdown table.

    python benchmarks/aggregate_results.py results/*.json --output BENCHMARKS.md
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def row_of(path: Path) -> dict | None:
    d = json.loads(path.read_text())
    c, m = d.get("config", {}), d.get("metrics", {})
    if not c.get("success", False) or "throughput" not in m:
        return None
    return {"framework": c.get("framework", "prime-rl"), "type": c.get("type"), "model": c.get("model_name"),
            "lora": c.get("lora_rank"), "seq_len": c.get("seq_len"), "gpus": c.get("num_gpus"),
            "device": c.get("device_name"), "ac": c.get("ac"), "attention": c.get("attention"),
            "tokens_per_s": m["throughput"]["mean"], "mfu": m.get("mfu", {}).get("mean"),
            "step_s": m.get("step_time", {}).get("mean"), "peak_gib": m.get("peak_memory", {}).get("gib")}


def table(rows: list[dict]) -> str:
    cols = ["framework", "type", "model", "lora", "seq_len", "gpus", "device", "ac", "attention", "tokens_per_s", "mfu",
            "step_s", "peak_gib"]
    out = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    for r in sorted(rows, key=lambda r: (str(r["model"]), str(r["type"]), r["gpus"] or 0, str(r["framework"]))):
        cells = [(f"{r[c]:.2f}" if isinstance(r[c], float) else str(r[c])) for c in cols]
        out.append("| " + " | ".join(cells) + " |")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    rows = [r for r in (row_of(Path(f)) for f in args.files) if r is not None]
    text = table(rows)
    if args.output:
        Path(args.output).write_text(text)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
