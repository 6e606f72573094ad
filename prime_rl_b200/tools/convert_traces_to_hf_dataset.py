"""Rollout traces of a run (``traces_*.jsonl`` chunks written by the file monitor) -> one
Parquet file that ``datasets.load_dataset("parquet", ...)`` reads
(reference: src/prime_rl/tools/convert_traces_to_hf_dataset.py).

    python -m prime_rl_b200.tools.convert_traces_to_hf_dataset <run_dir> <out.parquet> [--min-reward 0.5]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path


def collect(run_dir: Path, min_reward: float | None = None) -> list[dict]:
    rows = []
    for f in sorted(Path(run_dir).rglob("traces_*.jsonl")):
        if f.name == "traces_index.jsonl":
            continue
        with open(f) as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                try:
                    r = json.loads(line)
                except ValueError:
                    continue
                if min_reward is not None and float(r.get("reward", 0.0)) < min_reward:
                    continue
                rows.append({"env": r.get("env_name") or r.get("env"), "task_id": r.get("task_id"),
                             "reward": r.get("reward"), "advantage": r.get("advantage"),
                             "policy_version": r.get("policy_version"), "trace_id": r.get("trace_id"),
                             "prompt_ids": r.get("prompt_ids"), "completion_ids": r.get("completion_ids"),
                             "extra": json.dumps({k: v for k, v in r.items() if k not in
                                                  ("prompt_ids", "completion_ids")}, default=str)})
    return rows


def convert(run_dir: Path, out: Path, min_reward: float | None = None) -> int:
    import pyarrow as pa
    import pyarrow.parquet as pq

    rows = collect(run_dir, min_reward)
    out = Path(out)
    out.parent.mkdir(parents=True, exist_ok=True)
    pq.write_table(pa.Table.from_pylist(rows), str(out))
    return len(rows)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("run_dir", type=Path)
    ap.add_argument("out", type=Path)
    ap.add_argument("--min-reward", type=float, default=None)
    a = ap.parse_args(argv)
    print(f"wrote {convert(a.run_dir, a.out, a.min_reward)} rows to {a.out}")


if __name__ == "__main__":
    main()
