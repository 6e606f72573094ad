"""SFT trainer: token-weighted cross-entropy over packed rows, normalised by the *global*
number of loss tokens of the step (all-reduced), optional validation loop, checkpoints and
weight broadcasts for online evals (reference: src/prime_rl/trainer/sft/train.py)."""

from __future__ import annotations

import time
from pathlib import Path

import torch
import torch.distributed as dist

from ... import monitors as monitors_mod
from ...configs.sft import SFTConfig
from ...models import SeqInfo, apply_lora, build_model, resolve_arch
from ...parallel import get_parallel_dims, get_world, setup_distributed
from ...utils.logger import get_logger, setup_logger
from ..ckpt import CheckpointManager, Progress
from ..loss import shift_left
from ..optim import setup_optimizer
from ..perf import PerfCounter
from .data import setup_dataset


class SFTTrainer:
    def __init__(self, config: SFTConfig, device: torch.device | None = None):
        self.config = config
        self.world = get_world()
        self.device = device if device is not None else setup_distributed(timeout_seconds=config.dist_timeout_seconds)
        self.logger = get_logger()
        self.progress = Progress()
        self.run_dir = Path(config.output_dir) / (config.run.dir or config.run.name or "")

    def setup(self) -> "SFTTrainer":
        cfg, mc = self.config, self.config.model
        self.arch = resolve_arch(mc.name, mc.arch)
        if mc.debug.num_layers is not None:
            self.arch = self.arch.model_copy(update={"num_hidden_layers": mc.debug.num_layers})
        self.dims = get_parallel_dims(mc, self.world.world_size, is_moe=self.arch.is_moe,
                                      num_experts=self.arch.num_experts)
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = build_model(self.arch, device=self.device, dtype=dtype, attn_backend=mc.attn)
        p = Path(mc.name)
        if p.is_dir() and not mc.debug.random_init:
            from ..weights import load_hf_checkpoint

            load_hf_checkpoint(self.model, p)
        if mc.lora is not None:
            apply_lora(self.model, mc.lora.rank, mc.lora.alpha, mc.lora.target_modules, mc.lora.modules_to_save)
        from ...models import setup_quantization

        setup_quantization(self.model, mc, self.logger)
        if mc.ac is not None:
            self.model.ac_every = mc.ac.freq
            if mc.ac.mode == "selective":
                from ...ops.stash import kinds_from_targets

                self.model.ac_keep = kinds_from_targets(mc.ac.targets)
        self.model.train()
        multi = dist.is_initialized() and self.world.world_size > 1
        d = self.dims
        # context parallelism: the ranks of one replica read the same rows and each runs its chunk of every row
        self.cp_ctx, self.dp_rank, self.dp_size, self.cp_rank = None, self.world.rank, self.world.world_size, 0
        if d.cp_enabled:
            from ...models import check_context_parallel
            from ...parallel.cp import ContextParallel

            check_context_parallel(self.arch, d.cp, mc.cp_style)

            coords = d.coords(self.world.rank)
            self.dp_rank, self.cp_rank = coords["dp"], coords["cp"]
            self.dp_size = self.world.world_size // d.cp
            self.cp_ctx = ContextParallel(d.group("cp"), d.cp, self.cp_rank, style=mc.cp_style,
                                          fused_kv_gather=mc.cp_kv_exchange == "p2p", kv_exchange=mc.cp_kv_exchange)
        self.dp_group = d.group("dp_cp") if multi else None
        ep_on = d.ep_enabled and multi
        if ep_on:
            from ...parallel.ep import install_expert_parallel

            install_expert_parallel(self.model, d, mc.moe)
        # same sharding choices as the RL trainer: optimizer state partitioned (stage 2) or parameters too (stage 3)
        zero = multi and d.dp_shard_cp > 1 and mc.lora is None
        fsdp = None
        if zero and mc.zero_stage == 3:
            from ...parallel.fsdp import install_fsdp

            fsdp = install_fsdp(self.model, d.group("dp_shard_cp"), prefetch=mc.reshard_after_forward)
        self.optimizer = setup_optimizer(
            cfg.optim, self.model, max_steps=cfg.max_steps, scheduler_config=cfg.scheduler, dp_group=self.dp_group,
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
        # online evals: an evals process (or the launcher's inference server) follows the weights written here
        self.weight_sender = None
        if cfg.eval is not None or cfg.weight_broadcast is not None:
            from ...configs.trainer import FileSystemWeightBroadcastConfig
            from ...transports.weights import setup_weight_sender

            wb = cfg.weight_broadcast or FileSystemWeightBroadcastConfig()
            self.weight_sender = setup_weight_sender(wb, self.run_dir, self.world, self.model,
                                                     lora=mc.lora is not None, lora_cfg=mc.lora)
            self.broadcast_interval = cfg.eval.interval if cfg.eval is not None else 1
        self.monitor = monitors_mod.setup(cfg.monitors, self.run_dir, "trainer", is_master=self.world.is_master)
        self.ckpt = CheckpointManager(self.run_dir, cfg.ckpt, is_master=self.world.is_master, rank=self.world.rank) \
            if cfg.ckpt is not None or cfg.resume is not None else None
        self.dataset = setup_dataset(cfg.data, self.arch.vocab_size, self.dp_rank, self.dp_size)
        self.val_dataset = setup_dataset(cfg.val.data, self.arch.vocab_size, self.dp_rank, self.dp_size) \
            if cfg.val is not None else None
        if cfg.resume is not None and self.ckpt is not None:
            step = cfg.resume.step if cfg.resume.step is not None else self.ckpt.latest()
            if step is not None:
                self.ckpt.load(step, self.model, self.optimizer, self.progress, self.dataset)
                self.progress.step = step + 1
        self.data_iter = iter(self.dataset)
        self.micro_steps = max(1, cfg.data.batch_size // (cfg.data.micro_batch_size * self.dp_size))
        dev_name = torch.cuda.get_device_name(self.device) if self.device.type == "cuda" else "cpu"
        self.perf = PerfCounter(self.arch, cfg.data.seq_len, self.world.world_size, dev_name, lora=mc.lora is not None)
        return self

    def _row_loss(self, row: dict) -> tuple[torch.Tensor, torch.Tensor]:
        """Sum of the label NLL over loss tokens of one packed row, and the token count."""
        ids = row["input_ids"].to(self.device)
        mask = row["loss_mask"].to(self.device)
        seq = SeqInfo.from_lengths(row["sequence_lengths"], self.device)
        labels = shift_left(ids)
        lmask = shift_left(mask.to(torch.float32)).bool()        # position t predicts token t + 1
        # the last position of each document predicts the next document's first token: drop it
        ends = torch.tensor(row["sequence_lengths"], device=self.device).cumsum(0) - 1
        lmask[ends] = False
        if self.cp_ctx is not None:
            # every rank of the replica runs its chunk(s) of the row and sums the loss of its own tokens
            ids, labels, lm, seq = self.cp_ctx.shard_inputs(ids, labels, lmask.to(torch.float32), seq)
            lmask = lm.bool()
        hidden = self.model(ids, seq)
        lp, _ = self.model.logprobs_entropy(hidden, labels)
        return -(lp * lmask).sum(), lmask.sum()

    def step(self) -> dict:
        t0 = time.perf_counter()
        rows = [next(self.data_iter) for _ in range(self.micro_steps * self.config.data.micro_batch_size)]
        # global number of loss tokens of this step (same masks as _row_loss, computed on the host)
        exact = 0
        for r in rows:
            m = shift_left(r["loss_mask"].float()).bool()
            ends = torch.tensor(r["sequence_lengths"]).cumsum(0) - 1
            m[ends] = False
            exact += int(m.sum())
        if self.cp_rank != 0:
            exact = 0                                # the replica's rows are counted once
        count = torch.tensor([float(exact)], device=self.device)
        if self.dp_group is not None:
            dist.all_reduce(count, group=self.dp_group)
        denom = count.clamp_min(1.0)
        total = torch.zeros((), device=self.device)
        for r in rows:
            nll, _ = self._row_loss(r)
            (nll / denom.squeeze()).backward()
            total += nll.detach()
        self.optimizer.reduce_gradients()
        gnorm = self.optimizer.step()
        self.optimizer.zero_grad()
        if self.dp_group is not None:
            dist.all_reduce(total, group=self.dp_group)
        tokens = len(rows) * self.config.data.seq_len * self.dp_size
        self.progress.total_tokens += tokens
        dt = time.perf_counter() - t0
        tps = tokens / dt
        return {"loss": float(total / denom.squeeze()), "optim/grad_norm": float(gnorm), "optim/lr": self.optimizer.lr,
                "perf/throughput": tps, "perf/mfu": self.perf.mfu(tps), "time/step": dt, "loss_tokens": float(count)}

    @torch.no_grad()
    def validate(self, num_rows: int = 8) -> float:
        self.model.eval()
        it = iter(self.val_dataset)
        nll, cnt = torch.zeros((), device=self.device), torch.zeros((), device=self.device)
        for _ in range(num_rows):
            a, b = self._row_loss(next(it))
            nll += a
            cnt += b
        if self.dp_group is not None:
            dist.all_reduce(nll, group=self.dp_group)
            dist.all_reduce(cnt, group=self.dp_group)
        self.model.train()
        return float(nll / cnt.clamp_min(1))

    def run(self) -> None:
        cfg = self.config
        while cfg.max_steps is None or self.progress.step < cfg.max_steps:
            step = self.progress.step
            if self.val_dataset is not None and ((step == 0 and cfg.val.eval_on_start) or
                                                 (step > 0 and step % cfg.val.interval == 0)):
                self.monitor.log({"val/loss": self.validate()}, step)
            m = self.step()
            self.monitor.log(m, step)
            if self.world.is_master:
                self.logger.info(f"step {step} | loss {m['loss']:.4f} | grad_norm {m['optim/grad_norm']:.3f} | "
                                 f"{m['perf/throughput']:.0f} tok/s")
            if self.weight_sender is not None and (step + 1) % self.broadcast_interval == 0:
                t0 = time.perf_counter()
                self.weight_sender.broadcast(self.model, step)
                self.monitor.log({"time/broadcast_weights": time.perf_counter() - t0}, step)
            if self.ckpt is not None and cfg.ckpt is not None and cfg.ckpt.interval and \
                    (step + 1) % cfg.ckpt.interval == 0:
                self.ckpt.save(step, self.model, self.optimizer, self.progress, self.dataset)
                self.ckpt.maybe_clean()
            self.progress.step += 1
        self.monitor.finalize()


def train(config: SFTConfig) -> SFTTrainer:
    setup_logger(config.log.level, tag=f"sft:{get_world().rank}", json_logging=config.log.json_logging)
    t = SFTTrainer(config).setup()
    t.run()
    return t


def main(argv: list[str] | None = None) -> None:
    from ...configs.base import cli

    config = cli(SFTConfig, argv)
    if config.dry_run:
        print(config.to_json())
        return
    train(config)


if __name__ == "__main__":
    main()
