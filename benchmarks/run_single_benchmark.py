"""One training benchmark: a few RL or SFT optimizer steps on synthetic batches, summarised as a
JSON file with the layout of the reference's benchmark results
(``{"config": {...}, "metrics": {"mfu", "throughput", "step_time", "peak_memory"}}``;
reference: benchmarks/scripts/run_single_benchmark.py), so that results of both frameworks can
sit in one table (``aggregate_results.py``).

    python benchmarks/run_single_benchmark.py --type rl --model-name qwen3-30b-a3b --lora-rank 16 \
        --seq-len 16384 --num-gpus 1 --output result.json
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/run_single_benchmark.py --num-gpus 8 ...

Throughput is tokens per second over all GPUs, taken from the trainer's own per-step metrics
(``perf/throughput``), after ``--warmup`` untimed steps.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from datetime import datetime, timezone
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def _stats(xs: list[float]) -> dict:
    return {"mean": statistics.fmean(xs), "std": statistics.pstdev(xs) if len(xs) > 1 else 0.0, "min": min(xs),
            "max": max(xs)}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--type", default="rl", choices=["rl", "sft"])
    ap.add_argument("--num-gpus", type=int, default=1)
    ap.add_argument("--model-name", default="qwen3-0.6b")
    ap.add_argument("--lora-rank", default="full", help="'full' or an adapter rank")
    ap.add_argument("--seq-len", type=int, default=16384)
    ap.add_argument("--ac", default="Recompute", choices=["Recompute", "Offload", "None"])
    ap.add_argument("--attention", default="auto")
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--output", default="benchmark_result.json")
    ap.add_argument("--dry-run", action="store_true", help="print the trainer config and exit")
    return ap.parse_args(argv)


def build_config(args) -> dict:
    model = {"name": args.model_name, "seq_len": args.seq_len, "attn": args.attention, "cp": args.cp, "ep": args.ep,
             "ac": None if args.ac == "None" else {"mode": "full", "freq": 1}, "debug": {"random_init": True}}
    if args.ac == "Offload":
        model["ac_offloading"] = {"pin_memory": True}
    if args.lora_rank != "full":
        model["lora"] = {"rank": int(args.lora_rank), "alpha": 2.0 * int(args.lora_rank)}
    return {"model": model, "data": {"fake": {"batch_size": args.micro_batches * args.num_gpus}},
            "optim": {"type": "adamw", "lr": 1e-5}, "max_steps": None, "monitors": {"file": None},
            "output_dir": str(Path(args.output).resolve().parent / "benchmark_run"),
            "weight_broadcast": {"type": "filesystem"}}


def main(argv=None) -> int:
    args = parse_args(argv)
    cfg_dict = build_config(args)
    if args.dry_run:
        print(json.dumps(cfg_dict, indent=2))
        return 0
    import torch

    from prime_rl_b200.parallel import get_world

    world = get_world()
    if world.world_size != args.num_gpus:
        raise SystemExit(f"--num-gpus {args.num_gpus} but {world.world_size} ranks were launched (use torch.distributed.run)")
    t_start = time.time()
    result = {"config": {**{k.replace("-", "_"): v for k, v in vars(args).items()}, "framework": "prime_rl_b200",
                         "device_name": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu",
                         "timestamp": datetime.now(timezone.utc).isoformat(), "success": False, "error_reason": None},
              "metrics": {}}
    try:
        if args.type == "rl":
            from prime_rl_b200.configs.trainer import TrainerConfig
            from prime_rl_b200.trainer.rl.train import RLTrainer

            trainer = RLTrainer(TrainerConfig.model_validate(cfg_dict)).setup()
        else:
            from prime_rl_b200.configs.sft import SFTConfig
            from prime_rl_b200.trainer.sft.train import SFTTrainer

            sft = {**cfg_dict, "data": {"type": "fake", "seq_len": args.seq_len, "batch_size": args.micro_batches * args.num_gpus}}
            sft.pop("weight_broadcast", None)
            trainer = SFTTrainer(SFTConfig.model_validate(sft)).setup()
        rows = []
        for i in range(args.warmup + args.steps):
            m = trainer.step()
            if i >= args.warmup:
                rows.append(m)
        result["metrics"] = {
            "mfu": _stats([r.get("perf/mfu", 0.0) for r in rows]),
            "throughput": _stats([r["perf/throughput"] for r in rows]),
            "step_time": _stats([r["time/step"] for r in rows]),
        }
        if torch.cuda.is_available():
            peak = torch.cuda.max_memory_allocated() / 2 ** 30
            total = torch.cuda.get_device_properties(0).total_memory / 2 ** 30
            result["metrics"]["peak_memory"] = {"gib": peak, "pct": 100.0 * peak / total}
        result["config"]["success"] = True
    except Exception as e:  # the result file records the failure, as the reference's runner does
        result["config"]["error_reason"] = f"{type(e).__name__}: {e}"
    result["config"]["time_taken"] = time.time() - t_start
    if world.rank == 0:
        Path(args.output).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output).write_text(json.dumps(result, indent=2))
        print(json.dumps(result["metrics"]))
    return 0 if result["config"]["success"] else 1


if __name__ == "__main__":
    sys.exit(main())
