"""RL trainer: receives packed micro-batches, runs forward / fused logprob head / per-token
loss / backward / optimizer step, then offers the new weights to the inference engine.

``RLTrainer`` is the programmatic API (``setup()`` once, ``step()`` per optimizer step);
``train(config)`` is the loop the ``trainer`` entrypoint and ``torchrun -m
prime_rl_b200.trainer.rl.train @ trainer.toml`` run. Structure follows the reference's
``train()`` (src/prime_rl/trainer/rl/train.py:74-749).
"""

from __future__ import annotations

import gc
import math
import time
from pathlib import Path

import torch
import torch.distributed as dist

from ... import monitors as monitors_mod
from ...configs.trainer import TrainerConfig
from ...models import SeqInfo, apply_lora, build_model, freeze_router, resolve_arch
from ...parallel import get_parallel_dims, get_world, setup_distributed
from ...utils.logger import get_logger, setup_logger
from ..ckpt import CheckpointManager, Progress
from ..data import DataLoader, FakeDataLoader, TensorMicroBatch
from ..loss import compute_loss, setup_rl_loss_fn, shift_left, shift_right
from ..optim import setup_optimizer
from ..perf import PerfCounter
from ..stats import TensorStats


class RLTrainer:
    def __init__(self, config: TrainerConfig, device: torch.device | None = None):
        self.config = config
        self.world = get_world()
        self.device = device if device is not None else setup_distributed(timeout_seconds=config.dist_timeout_seconds)
        self.logger = get_logger()
        self.progress = Progress()
        self.run_dir = Path(config.output_dir)
        self.step_metrics: dict = {}

    # ------------------------------------------------------------------ setup
    def setup(self) -> "RLTrainer":
        cfg, mc = self.config, self.config.model
        self.arch = resolve_arch(mc.name, mc.arch)
        if mc.debug.num_layers is not None:
            self.arch = self.arch.model_copy(update={"num_hidden_layers": mc.debug.num_layers})
        self.dims = get_parallel_dims(mc, self.world.world_size, is_moe=self.arch.is_moe,
                                      num_experts=self.arch.num_experts)
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.monitor = monitors_mod.setup(cfg.monitors, self.run_dir, "trainer", is_master=self.world.is_master,
                                          run_config=cfg.model_dump(mode="json"))
        self.annotations = None
        if cfg.log_annotations:
            from .annotations import AnnotationWriter

            self.annotations = AnnotationWriter(self.monitor, self.world.rank, self.world.world_size)
        t0 = time.perf_counter()
        self.model = build_model(self.arch, device=self.device, dtype=dtype, attn_backend=mc.attn, seed=0)
        self._maybe_load_pretrained()
        self.mm = None
        if mc.vlm is not None:
            from ...models.vision import MultimodalLM, VisionConfig

            if not mc.vlm.freeze_vision_encoder:
                raise NotImplementedError("training the vision tower (set model.vlm.freeze_vision_encoder = true)")
            vc = VisionConfig(**{"out_hidden_size": self.arch.hidden_size, **mc.vlm.vision})
            self.mm = MultimodalLM(self.model, vc, mc.vlm.image_token_id, tuple(mc.vlm.mrope_section), dtype=dtype,
                                   device=self.device)
            for p in self.mm.visual.parameters():
                p.requires_grad_(False)
            if not mc.debug.random_init and Path(mc.name).is_dir():
                from ..weights import load_vision_tower

                n = load_vision_tower(self.mm.visual, Path(mc.name))
                self.logger.info(f"vision tower: {n} tensors from {mc.name}")
        if mc.debug.force_balanced_routing:
            for m in self.model.moe_layers():
                m.router.force_balanced = True
        if mc.lora is not None:
            adapted = apply_lora(self.model, mc.lora.rank, mc.lora.alpha, mc.lora.target_modules,
                                 mc.lora.modules_to_save, num_adapters=mc.lora.num_adapters)
            self.multi_lora = mc.lora.num_adapters > 1
            self.logger.info(f"LoRA r={mc.lora.rank} x {mc.lora.num_adapters} on {len(adapted)} modules")
        from ...models import setup_quantization

        setup_quantization(self.model, mc, self.logger)
        if mc.freeze_moe_router:
            freeze_router(self.model)
        if mc.ac is not None:
            self.model.ac_every = mc.ac.freq
            if mc.ac.mode == "selective":
                from ...ops.stash import kinds_from_targets

                self.model.ac_keep = kinds_from_targets(mc.ac.targets)
        self.model.train()
        self._setup_parallel()
        self.loss_fn = setup_rl_loss_fn(cfg.loss)
        d = self.dims
        multi = dist.is_initialized() and self.world.world_size > 1
        ep_on = d.ep_enabled and multi
        # Optimizer state is partitioned over the sharding ranks for full fine-tuning; LoRA
        # adapters are small and stay replicated.
        zero = multi and d.dp_shard_cp > 1 and mc.lora is None and not mc.fsdp_cpu_offload
        fsdp = None
        if zero and mc.zero_stage == 3:
            from ...parallel.fsdp import install_fsdp

            fsdp = install_fsdp(self.model, d.group("dp_shard_cp"), prefetch=mc.reshard_after_forward)
        self.optimizer = setup_optimizer(
            cfg.optim, self.model, max_steps=cfg.max_steps, scheduler_config=cfg.scheduler,
            dp_group=self.dp_cp_group,
            expert_reduce_group=d.group("ep_replicas") if ep_on else None,
            expert_norm_group=d.group("ep") if ep_on else None,
            shard_group=d.group("dp_shard_cp") if zero else None,
            replicate_group=d.group("dp_replicate") if (zero and d.dp_replicate > 1) else None,
            expert_shard_group=d.group("dp_shard_mod_ep")
            if (zero and ep_on and d.dp_replicate == 1 and d.dp_shard_cp // d.ep > 1) else None,
            offload="cpu" if mc.full_offload else ("state" if mc.optim_cpu_offload else None),
            offload_chunk=mc.full_offload.chunk_elements if mc.full_offload else 16 * 1024 * 1024,
            p2p_collectives=mc.optim_collectives == "p2p" and self.device.type == "cuda", fsdp=fsdp,
            offload_gradients=bool(mc.full_offload) and fsdp is not None,
            max_pinned_slots=mc.full_offload.max_pinned_slots if mc.full_offload else None)
        if mc.full_offload and mc.full_offload.numa_bind and self.device.type == "cuda":
            from ..optim_offload import bind_to_gpu_numa_node, pci_address

            node = bind_to_gpu_numa_node(pci_address(self.device))      # host buffers next to the GPU's PCIe root
            if node is not None:
                self.logger.info(f"CPU optimizer threads bound to NUMA node {node}")
        self.ckpt = CheckpointManager(self.run_dir, cfg.ckpt, is_master=self.world.is_master, rank=self.world.rank) \
            if cfg.ckpt is not None or cfg.resume is not None else None
        self._setup_data()
        self._maybe_resume()
        self.weight_sender = None
        if cfg.data.fake is None:
            from ...transports.weights import setup_weight_sender

            self.weight_sender = setup_weight_sender(cfg.weight_broadcast, self.run_dir, self.world, self.model,
                                                     lora=mc.lora is not None, lora_cfg=mc.lora)
        dev_name = torch.cuda.get_device_name(self.device) if self.device.type == "cuda" else "cpu"
        self.perf = PerfCounter(self.arch, mc.seq_len, self.world.world_size, dev_name, lora=mc.lora is not None)
        # distribution statistics over the loss tokens of all ranks (mean / median / std / min / max)
        self.token_stats = TensorStats(self.dp_cp_group)
        n_train = sum(p.numel() for p in self.model.parameters() if p.requires_grad)
        n_all = sum(p.numel() for p in self.model.parameters())
        self.logger.info(f"model {self.arch.model_type}: {n_all / 1e9:.2f}B params ({n_train / 1e6:.1f}M trainable), "
                         f"setup {time.perf_counter() - t0:.1f}s, dims {self.dims}")
        return self

    def close(self) -> None:
        """Releases what lives outside the tensor allocator (symmetric peer-memory buffers of the optimizer
        collectives, of the expert-parallel dispatcher and of context parallelism). Collective: every rank
        calls it. The trainer cannot step afterwards."""
        for g in getattr(self.optimizer, "groups", []):
            if g.p2p is not None:
                g.p2p.close()
                g.p2p = None
        if self.dims.ep_enabled:
            from ...parallel import ep_p2p

            ep_p2p.release_shared()
        if self.cp_ctx is not None and hasattr(self.cp_ctx, "close"):
            self.cp_ctx.close()

    def _maybe_load_pretrained(self) -> None:
        mc = self.config.model
        p = Path(mc.name)
        if mc.debug.random_init or not p.is_dir():
            return
        from ..weights import load_hf_checkpoint

        load_hf_checkpoint(self.model, p)

    def _setup_parallel(self) -> None:
        dims = self.dims
        self.dp_cp_group = dims.group("dp_cp") if dist.is_initialized() else None
        coords = dims.coords(self.world.rank)
        self.dp_rank, self.cp_rank = coords["dp"], coords["cp"]
        self.cp_ctx = None
        if dims.cp_enabled:
            from ...models import check_context_parallel
            from ...parallel.cp import ContextParallel

            check_context_parallel(self.arch, dims.cp, self.config.model.cp_style)

            self.cp_ctx = ContextParallel(dims.group("cp"), dims.cp, self.cp_rank, style=self.config.model.cp_style,
                                          fused_kv_gather=self.config.model.cp_kv_exchange == "p2p",
                                          kv_exchange=self.config.model.cp_kv_exchange)
        if dims.ep_enabled:
            from ...parallel.ep import install_expert_parallel

            install_expert_parallel(self.model, dims, self.config.model.moe)

    def _setup_data(self) -> None:
        cfg = self.config
        if cfg.data.fake is not None:
            self.dataloader = FakeDataLoader(cfg.data.fake.batch_size, cfg.model.seq_len, self.dims.dp, self.dp_rank,
                                             generate_samples=cfg.data.fake.generate_samples,
                                             vocab_size=min(self.arch.vocab_size, 120000))
        else:
            self.dataloader = DataLoader(self.run_dir, self.progress.step, self.dims.dp, self.dp_rank,
                                         cfg.rollout_transport)

    def _maybe_resume(self) -> None:
        cfg = self.config
        if cfg.resume is None or self.ckpt is None:
            return
        if cfg.resume.dir is not None:
            step, path = cfg.resume.dir_step, cfg.resume.dir / "trainer"
        else:
            step = cfg.resume.step if cfg.resume.step is not None else self.ckpt.latest()
            path = None
        if step is None:
            self.logger.warning("resume requested but no checkpoint found; starting fresh")
            return
        self.ckpt.load(step, self.model, self.optimizer, self.progress, self.dataloader, path=path)
        self.progress.step = step + 1 if not (cfg.ckpt and cfg.ckpt.skip_progress) else self.progress.step

    # ------------------------------------------------------------------ one micro-batch
    def forward_backward(self, mb: TensorMicroBatch, scales: tuple[float, float, float]) -> dict:
        dev = self.device
        mb = mb.to(dev)
        ids = mb.input_ids
        labels = shift_left(ids)
        inv_temp = 1.0 / mb.temperatures
        seq = SeqInfo(None, max(mb.sequence_lengths), mb.position_ids.to(torch.int32))
        cu = torch.zeros(len(mb.sequence_lengths) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(mb.sequence_lengths, dtype=torch.int32).cumsum(0)
        seq.cu_seqlens = cu.to(dev, non_blocking=True)
        if self.config.enable_router_replay:
            if mb.routed_experts is None:
                raise ValueError("router replay is enabled but the batch carries no routed_experts "
                                 "(enable return_routed_experts on the inference side)")
            seq.routed_experts = mb.routed_experts
        if self.cp_ctx is not None:
            ids, labels, inv_temp, seq = self.cp_ctx.shard_inputs(ids, labels, inv_temp, seq)
        offload = self.config.model.ac_offloading
        if offload is not None and dev.type == "cuda":
            from ...utils.act_offloading import OffloadActivations

            with OffloadActivations(pin_memory=offload.pin_memory, max_inflight=offload.max_inflight_activations):
                hidden = self._forward(ids, seq, mb)
        else:
            hidden = self._forward(ids, seq, mb)
        smask = None
        if mb.sampling_mask is not None:
            if self.cp_ctx is not None:
                raise NotImplementedError("sampling-mask replay together with context parallelism")
            sm = mb.sampling_mask                       # row t: the ids token t was drawn from
            smask = torch.cat([sm[1:], torch.full_like(sm[:1], -1)], dim=0)     # aligned with the labels
        logprobs, entropy = self.model.logprobs_entropy(hidden, labels, inv_temp, smask)
        if self.cp_ctx is not None:
            logprobs, entropy = self.cp_ctx.gather_outputs(logprobs, entropy)
        V = self.arch.vocab_size
        logprobs = shift_right(logprobs, math.log(1.0 / V))
        entropy = shift_right(entropy, math.log(float(V)))
        if self.annotations is not None:
            self.annotations.collect(mb, logprobs, entropy, self.progress.step)
        loss, lm = compute_loss(
            trainer_logprobs=logprobs, inference_logprobs=mb.inference_logprobs, advantages=mb.advantages,
            loss_mask=mb.loss_mask, rl_loss_fn=self.loss_fn, rl_scale=scales[0], ce_scale=scales[1],
            ref_kl_scale=scales[2], ref_logprobs=mb.ref_logprobs, rl_weights=mb.rl_weights, ce_weights=mb.ce_weights,
            ref_kl_weights=mb.ref_kl_weights, sequence_lengths=mb.sequence_lengths)
        loss.backward()
        mask = mb.loss_mask
        with torch.no_grad():
            # context-parallel ranks of one replica hold the same rows after the gather: only the first contributes
            own = mask if self.cp_rank == 0 else torch.zeros_like(mask)
            log_ratio = logprobs.detach() - mb.inference_logprobs
            self.token_stats.add("entropy", entropy, own)
            self.token_stats.add("mismatch_kl", torch.exp(log_ratio) - log_ratio - 1, own)
            self.token_stats.add("log_importance_ratio", log_ratio, own)
        out = {"loss": loss.detach(), "entropy": (entropy * mask).sum() / mask.sum().clamp_min(1)}
        out.update({k: v.detach() for k, v in lm.items()})
        return out

    def _forward(self, ids, seq, mb):
        """Decoder forward; multimodal rows go through the vision tower first."""
        if getattr(self, "multi_lora", False):
            from ...models.layers import set_lora_num_tokens

            set_lora_num_tokens(mb.lora_num_tokens)          # which adapter the tokens of this micro-batch use
        if self.mm is None:
            if mb.mm_kwargs:
                raise ValueError("the batch carries image tensors but the trainer has no model.vlm section")
            return self.model(ids, seq)
        if self.cp_ctx is not None:
            raise NotImplementedError("multimodal batches together with context parallelism")
        mm = mb.mm_kwargs or {}
        return self.mm(ids, seq, mm.get("pixel_values"), mm.get("image_grid_thw"))

    # ------------------------------------------------------------------ one optimizer step
    def step(self, micro_batches: list[TensorMicroBatch] | None = None) -> dict:
        t_start = time.perf_counter()
        if micro_batches is None:
            self.dataloader.wait_for_batch()
            t_wait = time.perf_counter() - t_start
            micro_batches = self.dataloader.get_batch()
        else:
            t_wait = 0.0
        counts = [0, 0, 0]
        for mb in micro_batches:
            for i, c in enumerate(mb.loss_token_counts()):
                counts[i] += c
        if dist.is_initialized() and self.world.world_size > 1:
            t = torch.tensor(counts, dtype=torch.int64, device=self.device)
            dist.all_reduce(t, group=self.dp_cp_group)
            if self.dims.cp > 1:
                t = t // self.dims.cp  # context-parallel ranks of a replica hold the same rows
            counts = t.tolist()
        scales = tuple(float(max(c, 1)) for c in counts)
        t_fb = time.perf_counter()
        agg: dict[str, list] = {}
        for mb in micro_batches:
            for k, v in self.forward_backward(mb, scales).items():
                agg.setdefault(k, []).append(v)
        if self.annotations is not None:
            self.annotations.flush()
        self.optimizer.reduce_gradients()
        grad_norm = self.optimizer.step()
        lr = self.optimizer.schedule.lr_at(self.optimizer.step_count - 1)
        self.optimizer.zero_grad()
        metrics = {k: torch.stack(v).sum() if k == "loss" else torch.stack(v).mean() for k, v in agg.items()}
        metrics["optim/grad_norm"] = grad_norm.reshape(())
        metrics.update({f"tokens/{k}": v for k, v in self.token_stats.compute().items()})
        metrics.update({f"moe/{k}": v for k, v in self.model.load_balance_stats().items()})
        # one device->host read for the whole step
        keys = list(metrics)
        vals = torch.stack([metrics[k].float().reshape(()) for k in keys]).cpu().tolist()
        out = dict(zip(keys, vals))
        tokens = sum(mb.num_tokens for mb in micro_batches) * self.dims.dp
        self.progress.total_tokens += tokens
        self.progress.total_samples += sum(len(mb.sequence_lengths) for mb in micro_batches) * self.dims.dp
        self.perf.count_tokens(tokens)
        now = time.perf_counter()
        out.update({"optim/lr": lr, "time/step": now - t_start, "time/wait_for_batch": t_wait,
                    "time/forward_backward": now - t_fb, "perf/tokens": tokens})
        tps = tokens / max(now - t_fb, 1e-9)
        out["perf/throughput"] = tps
        out["perf/throughput_per_gpu"] = tps / self.world.world_size
        out["perf/mfu"] = self.perf.mfu(tps)
        if self.device.type == "cuda":
            out["perf/peak_memory"] = torch.cuda.max_memory_allocated(self.device) / 2 ** 30
        self.step_metrics = out
        return out

    # ------------------------------------------------------------------ loop
    def run(self) -> None:
        cfg = self.config
        heartbeat = metrics_server = None
        if self.world.is_master and cfg.heartbeat is not None:
            from ...utils.heartbeat import Heartbeat

            heartbeat = Heartbeat(cfg.heartbeat.url)
        if self.world.is_master and cfg.metrics_server is not None:
            from ...utils.metrics_server import MetricsServer

            metrics_server = MetricsServer(cfg.metrics_server.port, cfg.metrics_server.host).start()
        if self.weight_sender is not None and self.progress.step > 0:
            # resumed run: re-seed the (stateless) inference engines with the restored policy; a
            # fresh run starts from weights both sides already share
            self.weight_sender.broadcast(self.model, self.progress.step - 1)
        profiler = None
        if cfg.trace_path is not None:
            # torch.profiler trace (CPU + CUDA activities) of the whole run, one file per rank
            # (reference: trainer/rl/train.py:243-247, 724-730; meant for runs of a few steps)
            from torch.profiler import ProfilerActivity, profile

            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.device.type == "cuda" else [])
            profiler = profile(activities=acts, record_shapes=True)
            profiler.__enter__()
        if cfg.memory_profiler_path is not None and self.device.type == "cuda":
            torch.cuda.memory._record_memory_history(max_entries=100000)
        while cfg.max_steps is None or self.progress.step < cfg.max_steps:
            step = self.progress.step
            m = self.step()
            if cfg.memory_profiler_path is not None and self.device.type == "cuda":
                out = Path(cfg.memory_profiler_path)
                out.mkdir(parents=True, exist_ok=True)
                torch.cuda.memory._dump_snapshot(str(out / f"rank_{self.world.rank}_step_{step}.pickle"))
            # the weights of the last step have no taker in an in-memory transport: the orchestrator stops after
            # shipping the batch for it, and a sender that waits for an acknowledgement would wait out its timeout
            last = cfg.max_steps is not None and step + 1 >= cfg.max_steps
            if self.weight_sender is not None and not (last and getattr(self.weight_sender, "require_ack", False)):
                t0 = time.perf_counter()
                self.weight_sender.broadcast(self.model, step)
                m["time/broadcast_weights"] = time.perf_counter() - t0
            if self.ckpt is not None and cfg.ckpt is not None and cfg.ckpt.interval and \
                    (step + 1) % cfg.ckpt.interval == 0:
                t0 = time.perf_counter()
                self.ckpt.save(step, self.model, self.optimizer, self.progress, self.dataloader)
                self.ckpt.maybe_clean()
                m["time/save_ckpt"] = time.perf_counter() - t0
            self.monitor.log(m, step)
            if metrics_server is not None:
                metrics_server.update(m, step)
            if heartbeat is not None:
                heartbeat.beat()
            if self.world.is_master:
                self.logger.info(f"step {step} | loss {m['loss']:.4f} | entropy {m.get('entropy', 0):.3f} | "
                                 f"grad_norm {m['optim/grad_norm']:.3f} | {m['perf/throughput']:.0f} tok/s | "
                                 f"mfu {m['perf/mfu']:.1f}% | {m['time/step']:.2f}s")
            self.progress.step += 1
            if cfg.gc is not None and self.progress.step % cfg.gc.interval == 0:
                gc.collect()
        if self.ckpt is not None and cfg.ckpt is not None and self.progress.step > 0:
            last = self.progress.step - 1
            if last not in self.ckpt.saved_steps:
                self.ckpt.save(last, self.model, self.optimizer, self.progress, self.dataloader)
        if profiler is not None:
            profiler.__exit__(None, None, None)
            out = Path(cfg.trace_path)
            out.mkdir(parents=True, exist_ok=True)
            profiler.export_chrome_trace(str(out / f"trace_{self.world.rank}.json.gz"))
        self.monitor.finalize()
        if metrics_server is not None:
            metrics_server.stop()


def train(config: TrainerConfig) -> RLTrainer:
    setup_logger(config.log.level, tag=f"trainer:{get_world().rank}", json_logging=config.log.json_logging)
    trainer = RLTrainer(config).setup()
    trainer.run()
    return trainer


def main(argv: list[str] | None = None) -> None:
    from ...configs.base import cli

    config = cli(TrainerConfig, argv)
    if config.dry_run:
        print(config.to_json())
        return
    train(config)
    from ...parallel.world import cleanup

    cleanup()


if __name__ == "__main__":
    main()
