"""Headline benchmark: RL trainer tokens/s and rollout decode tokens/s on the Qwen3-30B-A3B shape.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Trainer (``value``). Two configurations; ``--mode auto`` (the default) picks by what fits:

  full   the headline one: full fine-tuning, expert parallelism over all N GPUs (every rank owns
         128 / N experts; tokens travel through the peer-memory dispatcher), optimizer state of the
         dense parameters partitioned over the ranks with its reduce-scatter / all-gather as
         peer-memory kernels, full activation recomputation, packed rows of 8192 tokens, 64 rows per
         optimizer step for the whole job (64 / N micro-batches per GPU: the total work is fixed,
         strong scaling). Needs fp32 master + moments + gradients of 30.5 B parameters spread over
         the GPUs: N >= 4.
  lora   the reference's published 8xB200 row for this model: LoRA rank 16 on attention
         projections and experts, 16384-token rows, 2 micro-batches per GPU and step (weak
         scaling), frozen base replicated, adapter gradients all-reduced. Used where ``full``
         does not fit (the line then says ``"config_3": "does not fit"``), and always reported
         under ``lora_dp`` next to a ``full`` result so that both numbers stay comparable over time.

Two passes of K steps each are timed after W warm-up steps:
  * ``value``  device time (CUDA events, max over ranks) with the step's inputs already on
    the device;
  * ``e2e``    wall clock through ``RLTrainer.step()`` fed by the data loader: pinned host
    batches -> device every step, loss / metrics read back every step.

Rollout (``rollout_decode``): the engine with block-scaled fp8 weights (128 x 128 weight blocks,
1 x 128 activation scales) and a bf16 paged KV cache of 16-token pages, tensor-parallel over up
to 4 GPUs (the shape has 4 KV heads) with data-parallel groups beyond that, 256 concurrent
requests per group = 32 prompts of 1024 tokens x 8 samples that share the prompt's pages through
the prefix cache, temperature 1.0. Decode steps are timed at the contexts a 4096-token generation
passes through (1024, 3072, 5120 tokens), then one full weight push bf16 -> fp8 in flight.

Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import faulthandler
import gc
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
faulthandler.enable()          # a native crash leaves the Python stack of every thread on stderr
sys.path.insert(0, str(ROOT))

# reference, 8xB200, Qwen3-30B-A3B RL LoRA r16, seq 16384 (benchmarks/results/BENCHMARKS.md:60): its only
# successful 8xB200 run of this model (the full fine-tuning runs of the same table failed on B200)
BASELINE_TPS_8GPU = 9266.4


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--mode", default="auto", choices=["auto", "lora", "full"])
    ap.add_argument("--seq-len", type=int, default=None, help="tokens per packed row (default: 8192 full, 16384 lora)")
    ap.add_argument("--rows", type=int, default=64, help="full mode: rows per optimizer step over the whole job")
    ap.add_argument("--micro-batches", type=int, default=2, help="lora mode: micro-batches per GPU and step")
    ap.add_argument("--dispatch", default="p2p", choices=["p2p", "torch"], help="full mode: expert-parallel dispatcher")
    ap.add_argument("--optim-collectives", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--zero-stage", type=int, default=None, choices=[2, 3],
                    help="full mode: 3 = parameters sharded per layer (the default for dense models), 2 = replicated")
    ap.add_argument("--cp", type=int, default=1, help="full mode: context-parallel ranks per replica (long rows)")
    ap.add_argument("--cp-style", default="ring", choices=["ring", "ulysses"])
    ap.add_argument("--layers", type=int, default=None, help="debug: truncate the model (result is not a bench value)")
    ap.add_argument("--attn", default="auto")
    ap.add_argument("--no-rollout-decode", action="store_true", help="skip the rollout measurement")
    ap.add_argument("--no-secondary", action="store_true", help="full mode: skip the LoRA / data-parallel comparison run")
    ap.add_argument("--rollout-contexts", default="1024,3072,5120")
    ap.add_argument("--rollout-steps", type=int, default=16)
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


def full_fit(arch, n: int, total_bytes: int) -> tuple[bool, float]:
    """Does full fine-tuning with experts and optimizer state spread over ``n`` GPUs fit in one GPU's
    memory? Per parameter: 2 B bf16 value + 4 B flat fp32 gradient on every holder, 12 B master + moments
    (+ 4 B reduced gradient slice for the partitioned dense part) on its owner."""
    from prime_rl_b200.trainer.perf import count_params

    dense, expert = count_params(arch)
    per_gpu = 6 * (dense + expert / n) + 12 * (dense + expert) / n + 4 * dense / n
    need = per_gpu + 14e9            # activations, logits gradient chunk, dispatch buffers, allocator slack
    return need <= 0.93 * total_bytes, need / 1e9


def trainer_pass(args, mode: str, world, steps: int, warmup: int, want_e2e: bool = True) -> dict:
    """Builds the trainer for ``mode``, times it and tears it down again. Collective: every rank calls."""
    import torch
    import torch.distributed as dist

    from prime_rl_b200.configs.trainer import TrainerConfig
    from prime_rl_b200.ops import _runtime as rt
    from prime_rl_b200.trainer.rl.train import RLTrainer

    n = world.world_size
    if mode == "full":
        from prime_rl_b200.models import resolve_arch

        moe = resolve_arch(args.model).is_moe
        seq_len = args.seq_len or 8192
        cp = max(1, args.cp)
        replicas = max(1, n // cp)
        per_gpu = max(1, args.rows // replicas)          # micro-batches per replica and step
        global_rows = per_gpu * replicas
        mcfg = {"name": args.model, "seq_len": seq_len, "attn": args.attn, "ac": {"mode": "full", "freq": 1},
                "optim_collectives": args.optim_collectives,
                "debug": {"random_init": True, "num_layers": args.layers}}
        if cp > 1:
            mcfg.update(cp=cp, cp_style=args.cp_style)
        if moe:
            mcfg.update(ep=n if n > 1 else 1,
                        moe={"dispatch": {"type": args.dispatch} if args.dispatch == "torch" else
                             {"type": "p2p", "capacity_factor": float(min(n, 4))}})       # receive buffers for 4x the
            # balanced share. The default (the worst case, ep x) makes the buffers twice as long at 8 GPUs, and the
            # elementwise kernels of the expert path walk whole buffers: measured 5.74 s per step against 5.44 s
            par = (f"ep{n} (128/{n} experts per GPU, peer-memory dispatch) x zero{n} (dense optimizer state "
                   f"partitioned, {args.optim_collectives} reduce-scatter / all-gather)") if n > 1 else "single GPU"
        else:
            zs = args.zero_stage or (3 if n > 1 else 2)
            mcfg.update(ep=1, zero_stage=zs)
            if zs == 3:
                mcfg["optim_collectives"] = "nccl"       # the per-layer collectives of the sharding runtime
            par = (f"zero{zs} over {n} GPUs" + (" (parameters, gradients and optimizer state sharded per layer, "
                                                 "next layer gathered ahead)" if zs == 3 else "")) if n > 1 \
                else "single GPU"
            if cp > 1:
                par += f", cp{cp} ({args.cp_style}, zig-zag)"
        scaling = "strong"
    else:
        seq_len = args.seq_len or 16384
        per_gpu = args.micro_batches
        global_rows = per_gpu * n
        mcfg = {"name": args.model, "seq_len": seq_len, "attn": args.attn, "ac": {"mode": "full", "freq": 1},
                "ep": 1, "lora": {"rank": 16, "alpha": 32.0}, "debug": {"random_init": True, "num_layers": args.layers}}
        scaling = "weak"
        par = f"dp{n} (frozen base replicated, adapter grads all-reduced)"
    cfg = TrainerConfig.model_validate({
        "model": mcfg, "data": {"fake": {"batch_size": global_rows}},
        "optim": {"type": "adamw", "lr": 1e-5, "weight_decay": 0.01, "max_norm": 1.0},
        "max_steps": None, "output_dir": str(Path(tempfile.gettempdir()) / f"prime_rl_b200_bench_{mode}"),
        "monitors": {"file": None}, "weight_broadcast": {"type": "filesystem"}})
    trainer = RLTrainer(cfg).setup()
    dev = trainer.device
    tokens_per_step = global_rows * seq_len

    def sync():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        trainer.step()
    rt.check_status()
    sync()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    # ---- pass A: device time, inputs pre-staged on the device
    staged = [[mb.to(dev) for mb in trainer.dataloader.get_batch()] for _ in range(steps)]
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
    # ---- pass B: end to end through the public API
    h2d = d2h = 0
    e2e_s = float("nan")
    if want_e2e:
        sync()
        t0 = time.perf_counter()
        for _ in range(steps):
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
    value = tokens_per_step * steps / (dev_ms / 1e3)
    out = {"mode": mode, "value": value, "ms_per_step": dev_ms / steps, "tokens_per_step": tokens_per_step,
           "seq_len": seq_len, "global_rows": global_rows, "rows_per_gpu": per_gpu, "scaling": scaling,
           "parallelism": par, "clocks": clocks, "gpu_launches": launches, "loss": m.get("loss"),
           "mfu_percent": trainer.perf.mfu(value), "peak_memory_gib": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
           "e2e": None if not want_e2e else {"value": tokens_per_step * steps / e2e_s, "unit": "tokens/s",
                                            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}}
    # ---- tear down: the next phase needs the memory (symmetric buffers are outside torch's allocator)
    trainer.close()
    del trainer, mbs, m
    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats(dev)
    sync()
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) == 0:
            reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from prime_rl_b200.models import resolve_arch
    from prime_rl_b200.parallel import get_world, setup_distributed
    from prime_rl_b200.utils.logger import setup_logger

    world = get_world()
    n = world.world_size
    setup_logger("warning" if world.rank else "info", tag=f"bench:{world.rank}")
    dev = setup_distributed()
    arch = resolve_arch(args.model)
    if args.layers:
        arch = arch.model_copy(update={"num_hidden_layers": args.layers})
    fits, need_gb = full_fit(arch, n, torch.cuda.get_device_properties(dev).total_memory)
    mode = args.mode
    if mode == "auto":
        mode = "full" if (fits and (n > 1 or not arch.is_moe)) else "lora"
    primary = trainer_pass(args, mode, world, args.steps, args.warmup)
    secondary = None
    if mode == "full" and not args.no_secondary:
        try:
            s = trainer_pass(args, "lora", world, min(args.steps, 3), 3, want_e2e=False)
            secondary = {k: s[k] for k in ("value", "ms_per_step", "seq_len", "global_rows", "scaling", "parallelism",
                                           "mfu_percent", "peak_memory_gib")}
            secondary["metric"] = "RL trainer tokens/s, LoRA r16, data parallel (the reference's published B200 row)"
            secondary["vs_baseline"] = s["value"] / (BASELINE_TPS_8GPU * n / 8)
        except Exception as e:      # the headline number stands on its own
            secondary = {"error": f"{type(e).__name__}: {e}"[:300]}

    rollout = None
    if not args.no_rollout_decode:
        try:
            from prime_rl_b200.engine.bench_decode import run_rollout_bench

            rollout = run_rollout_bench(args.model, contexts=[int(c) for c in args.rollout_contexts.split(",")],
                                        steps=args.rollout_steps, layers=args.layers, dev=dev)
        except Exception as e:
            err = f"{type(e).__name__}: {e}"[:300]
            rollout = {"error": err}
    if world.rank == 0:
        p = primary
        headline = args.model == "qwen3-30b-a3b"        # the published reference row is for this shape only
        line = {
            "metric": "RL trainer tokens/s, Qwen3-30B-A3B shape" if headline else f"RL trainer tokens/s, {args.model} shape",
            "value": p["value"], "unit": "tokens/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": p["ms_per_step"],
            "higher_is_better": True, "scaling": p["scaling"],
            "vs_baseline": p["value"] / (BASELINE_TPS_8GPU * n / 8) if headline else None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": args.model if args.layers is None else f"{args.model}[{args.layers} layers: debug]",
                       "mode": "rl-full" if p["mode"] == "full" else "rl-lora-r16",
                       "global_batch": p["global_rows"], "seq_len": p["seq_len"], "rows_per_gpu": p["rows_per_gpu"],
                       "parallelism": p["parallelism"], "activation_checkpointing": "full", "loss": "ipo",
                       "optimizer": "adamw",
                       "l2": "inputs, activations and weights exceed L2 many times over; no flush between steps",
                       "vs_baseline_note": "reference 9266 tok/s (LoRA r16, seq 16384, 8 GPUs; its full fine-tuning runs "
                                           "failed on B200), scaled by n_gpus/8"},
            "clocks": p["clocks"], "e2e": p["e2e"], "gpu_launches": p["gpu_launches"], "loss": p["loss"],
            "mfu_percent": p["mfu_percent"], "peak_memory_gib": p["peak_memory_gib"],
            "rollout_decode": rollout,
        }
        if p["mode"] == "full":
            line["lora_dp"] = secondary
        else:
            line["config_3"] = ("does not fit" if not fits else "not selected") + \
                f": full fine-tuning of this shape needs about {need_gb:.0f} GB per GPU at N = {n}"
        print(json.dumps(line))
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
