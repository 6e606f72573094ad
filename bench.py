"""Headline benchmark: RL trainer tokens/s on the Qwen3-30B-A3B shape.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (the reference's own published 8xB200 row for this model): RL step, LoRA rank 16 on
attention projections and experts, full activation recomputation, packed sequences of
16384 tokens, 2 micro-batches per GPU and step, bf16, synthetic token ids, random-init
weights. Weak scaling: per-GPU work is fixed, the frozen base weights are replicated
(61 GB of the 180 GB) and only the adapter gradients are all-reduced.

Two passes of K steps each are timed after W warm-up steps:
  * ``value``  device time (CUDA events, max over ranks) with the step's inputs already on
    the device;
  * ``e2e``    wall clock through ``RLTrainer.step()`` fed by the data loader: pinned host
    batches -> device every step, loss / metrics read back every step.
Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BASELINE_TPS_8GPU = 9266.4  # reference, 8xB200, Qwen3-30B-A3B RL LoRA r16, seq 16384 (benchmarks/results/BENCHMARKS.md:60)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--seq-len", type=int, default=16384)
    ap.add_argument("--micro-batches", type=int, default=2, help="micro-batches per GPU and step")
    ap.add_argument("--mode", default="lora", choices=["lora", "full"])
    ap.add_argument("--layers", type=int, default=None, help="debug: truncate the model (result is not a bench value)")
    ap.add_argument("--attn", default="auto")
    ap.add_argument("--no-rollout-decode", action="store_true",
                    help="skip the second measurement (rollout decode tokens/s of the engine, one replica per GPU)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock, power and throttle reasons of this process's GPU during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc, self.thread = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples is "under load"
        sm_load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(sm_load) if sm_load else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    # The one offline install (`pip install --no-index --no-build-isolation --find-links
    # /opt/wheelhouse --target baseline/_ref <reference>`) fails: the reference's build backend
    # (hatchling) is neither in the image nor in the wheelhouse, so no wheel can be built.
    ref = ROOT / "baseline" / "_ref" / "prime_rl"
    reason = "reference not installable offline: build backend 'hatchling' missing from image and wheelhouse"
    if ref.exists():
        reason = "reference package present but its dependencies (verifiers, renderers, torch>=2.13, vllm 0.28) are not installed"
    print(json.dumps({"impl": "reference", "unavailable": reason}))


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) == 0:
            reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from prime_rl_b200.configs.trainer import TrainerConfig
    from prime_rl_b200.ops import _runtime as rt
    from prime_rl_b200.parallel import get_world
    from prime_rl_b200.trainer.rl.train import RLTrainer
    from prime_rl_b200.utils.logger import setup_logger

    world = get_world()
    n = world.world_size
    setup_logger("warning" if world.rank else "info", tag=f"bench:{world.rank}")
    mcfg = {"name": args.model, "seq_len": args.seq_len, "attn": args.attn, "ac": {"mode": "full", "freq": 1},
            "ep": 1, "debug": {"random_init": True, "num_layers": args.layers}}
    if args.mode == "lora":
        mcfg["lora"] = {"rank": 16, "alpha": 32.0}
    cfg = TrainerConfig.model_validate({
        "model": mcfg, "data": {"fake": {"batch_size": args.micro_batches * n}},
        "optim": {"type": "adamw", "lr": 1e-5, "weight_decay": 0.01, "max_norm": 1.0},
        "max_steps": None, "output_dir": str(Path(tempfile.gettempdir()) / "prime_rl_b200_bench_run"), "monitors": {"file": None},
        "weight_broadcast": {"type": "filesystem"}})
    trainer = RLTrainer(cfg).setup()
    dev = trainer.device
    tokens_per_step = args.micro_batches * args.seq_len * n

    def sync():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------ warm-up (shared by both passes)
    for _ in range(args.warmup):
        trainer.step()
    rt.check_status()
    sync()

    sampler = ClockSampler(dev.index or 0)
    sampler.start()

    # ------------------------------------------------------------ pass A: device time, inputs pre-staged
    staged = [[mb.to(dev) for mb in trainer.dataloader.get_batch()] for _ in range(args.steps)]
    sync()
    launches0 = rt.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for mbs in staged:
        m = trainer.step(mbs)
    ev1.record()
    sync()
    dev_ms = ev0.elapsed_time(ev1)
    launches = rt.launch_count() - launches0
    del staged

    # ------------------------------------------------------------ pass B: end to end through the public API
    h2d = d2h = 0
    sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        mbs = trainer.dataloader.get_batch()           # pinned host memory
        h2d = sum(mb.h2d_bytes() for mb in mbs)
        m = trainer.step(mbs)                          # H2D copies + one D2H read of the step's metrics
        d2h = 4 * len([k for k in m if not k.startswith(("time/", "perf/", "optim/lr"))])
    sync()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    rt.check_status()

    t = torch.tensor([dev_ms, e2e_s], dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s = t.tolist()
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e = tokens_per_step * args.steps / e2e_s
    loss_value, mfu, peak_gib = m.get("loss"), trainer.perf.mfu(value), torch.cuda.max_memory_allocated(dev) / 2 ** 30

    # ------------------------------------------------------------ second number of the headline: rollout decode
    # One engine replica per GPU (data-parallel serving), 256 requests of 1024 prompt tokens each, 16 timed
    # decode steps through Engine.step; aggregate tokens/s = sum over replicas, step time = slowest replica.
    rollout = None
    if not args.no_rollout_decode:
        import gc
        import math

        local, err = [float("nan"), float("nan")], None
        try:
            from prime_rl_b200.engine.bench_decode import run_decode

            del trainer, mbs
            gc.collect()
            torch.cuda.empty_cache()
            r = run_decode(args.model, batch=256, prompt=1024, steps=16, warmup=4, layers=args.layers, dev=dev)
            local = [r["decode_tokens_per_s"], r["ms_per_step"]]
        except Exception as e:  # the trainer number stands on its own
            err = f"{type(e).__name__}: {e}"[:300]
        t = torch.tensor(local, dtype=torch.float64, device=dev)
        if n > 1:                                   # every rank takes part, whatever happened to its own replica
            tot = t.clone()
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t[0] = tot[0]
        if math.isnan(float(t[0])) or math.isnan(float(t[1])):
            rollout = {"error": err or "an engine replica on another rank failed"}
        else:
            rollout = {"metric": "rollout decode tokens/s", "value": float(t[0]), "unit": "tokens/s",
                       "ms_per_step": float(t[1]), "batch_per_gpu": 256, "prompt_len": 1024, "steps": 16,
                       "parallelism": f"dp{n} (one engine replica per GPU)", "cuda_graphs": True, "dtype": "bf16"}
    if world.rank == 0:
        print(json.dumps({
            "metric": "RL trainer tokens/s, Qwen3-30B-A3B shape", "value": value, "unit": "tokens/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / (BASELINE_TPS_8GPU * n / 8),
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": args.model if args.layers is None else f"{args.model}[{args.layers} layers: debug]",
                       "mode": f"rl-{args.mode}" + ("-r16" if args.mode == "lora" else ""),
                       "global_batch": args.micro_batches * n, "seq_len": args.seq_len,
                       "parallelism": f"dp{n}" + (" (frozen base replicated, adapter grads all-reduced)"
                                                   if args.mode == "lora" else ""),
                       "activation_checkpointing": "full", "loss": "ipo", "optimizer": "adamw",
                       "l2": "inputs and weights (61 GB) exceed L2; no flush between steps",
                       "vs_baseline_note": "reference 9266 tok/s on 8 GPUs, scaled by n_gpus/8"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "loss": loss_value, "mfu_percent": mfu,
            "peak_memory_gib": peak_gib, "rollout_decode": rollout,
        }))
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
