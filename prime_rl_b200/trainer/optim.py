"""Optimizers on flat buffers.

All trainable parameters of a model are re-homed into ONE contiguous buffer in the compute
dtype (the parameters become views of it); next to it live an fp32 master copy, fp32
gradient accumulator and the optimizer moments, all flat and equally long. A step is then
a handful of launches regardless of the parameter count:

    sum of squares -> clip coefficient (on device) -> fused update (master, moments, compute copy)

and the data-parallel gradient reduction is a single collective over the flat accumulator.
The learning rate and bias corrections are read from device memory by the kernel, so the
whole step is free of host synchronisation and can be captured in a CUDA graph.

Covers the reference's SGD / AdamW / SignSGD / Muon choices
(src/prime_rl/trainer/optim/__init__.py:102-249) and its LR schedules
(src/prime_rl/trainer/scheduler.py).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import optim as optim_ops


@dataclass
class ParamSlot:
    name: str
    offset: int
    numel: int
    shape: torch.Size


class FlatBuffers:
    """Owns the flat parameter / master / gradient storage of a set of parameters."""

    def __init__(self, named_params: list[tuple[str, torch.nn.Parameter]], master_dtype=torch.float32,
                 align: int = 8, pad_to: int = 1, full_master: bool = True, alloc=None):
        """``alloc(numel, dtype) -> (flat, grad)`` supplies the two flat tensors (zero-filled) when they
        have to live in special memory (the peer-memory collectives keep them in a symmetric buffer)."""
        params = [(n, p) for n, p in named_params if p.requires_grad]
        if not params:
            raise ValueError("no trainable parameters")
        self.device = params[0][1].device
        self.dtype = params[0][1].dtype
        self.slots: list[ParamSlot] = []
        off = 0
        for n, p in params:
            if p.dtype != self.dtype:
                raise ValueError(f"mixed parameter dtypes ({n}: {p.dtype} vs {self.dtype})")
            self.slots.append(ParamSlot(n, off, p.numel(), p.shape))
            off += (p.numel() + align - 1) // align * align
        off = (off + pad_to - 1) // pad_to * pad_to
        self.numel = off
        self.params = [p for _, p in params]
        given_grad = None
        if alloc is not None:
            self.flat, given_grad = alloc(off, self.dtype)
        else:
            self.flat = torch.zeros(off, dtype=self.dtype, device=self.device)
        for s, p in zip(self.slots, self.params):
            view = self.flat[s.offset:s.offset + s.numel].view(s.shape)
            view.copy_(p.data)
            p.data = view
        if not full_master:
            self.master = None          # the owner keeps a sharded master copy instead
        elif self.dtype == master_dtype:
            self.master = self.flat
        else:
            self.master = self.flat.to(master_dtype)
        self.grad = given_grad if given_grad is not None else torch.zeros(off, dtype=torch.float32, device=self.device)
        self._grad_views = [self.grad[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots]

    @property
    def has_lowp(self) -> bool:
        return self.master is not None and self.master is not self.flat

    def accumulate_grads(self) -> None:
        """grad_acc += p.grad (fp32) for every parameter, then drops p.grad."""
        for p, gv in zip(self.params, self._grad_views):
            if p.grad is not None:
                gv.add_(p.grad)
                p.grad = None

    def install_hooks(self) -> None:
        """Accumulate into the flat fp32 buffer as soon as autograd produced a gradient, so
        that low-precision per-parameter gradients never pile up across micro-batches."""
        for p, gv in zip(self.params, self._grad_views):
            def hook(param, gv=gv):
                if param.grad is None:          # the weight-gradient GEMM already added its product to ``gv``
                    return
                gv.add_(param.grad)
                param.grad = None
            p.register_post_accumulate_grad_hook(hook)
            if p.is_cuda and p.dim() >= 2:
                # the weight-gradient GEMMs of ops/matmul.py add straight into this view (no bf16 gradient, no
                # second pass); gradients that still arrive through autograd take the hook above
                p._grad_acc = gv

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p in self.params:
            p.grad = None

    def sync_from_master(self) -> None:
        if self.has_lowp:
            self.flat.copy_(self.master)

    def named_views(self, flat: torch.Tensor) -> dict[str, torch.Tensor]:
        return {s.name: flat[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots}


class LRSchedule:
    """Closed-form learning-rate schedules (constant, linear warmup-stable-decay, cosine)."""

    def __init__(self, config, max_steps: int | None, lr: float):
        self.config, self.max_steps, self.base_lr = config, max_steps, lr

    def lr_at(self, step: int) -> float:
        """Learning rate used by the ``step``-th optimizer step (0-based)."""
        c, lr = self.config, self.base_lr
        t = getattr(c, "type", "constant")
        if t == "constant":
            return lr
        min_factor = (c.min_lr / lr) if (c.min_lr > 0 and lr > 0) else 1e-8
        warm = c.warmup_steps
        if warm > 0 and step < warm:
            return lr * (min_factor + (1.0 - min_factor) * step / warm)
        if t == "linear":
            if c.decay_steps > 0:
                start = self.max_steps - c.decay_steps
                if step >= start:
                    frac = min(1.0, (step - start) / max(1, c.decay_steps - 1))
                    return lr * (1.0 + (min_factor - 1.0) * frac)
            return lr
        if t == "cosine":
            total = max(1, self.max_steps - warm)
            prog = min(1.0, (step - warm) / total)
            return c.min_lr + (lr - c.min_lr) * 0.5 * (1.0 + math.cos(math.pi * prog))
        raise ValueError(f"unknown scheduler type {t}")


def newton_schulz(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation used by Muon (bf16 on GPU). 2-D matrices on the GPU run on the
    tcgen05 GEMM with the polynomial's additions folded into its epilogue (``alpha * A.B + beta * C``): three
    launches per iteration and no separate element-wise pass; stacked (expert) matrices use batched matmul."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.to(torch.bfloat16 if g.is_cuda else torch.float32)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-2, -1)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    if x.is_cuda and x.dim() == 2 and x.shape[0] % 8 == 0 and x.shape[1] % 8 == 0:
        from ..ops.matmul import gemm

        x = x.contiguous()
        for _ in range(steps):
            A = gemm(x, x)                                   # x x^T (symmetric)
            B = A.clone()
            gemm(A, A, out=B, alpha=c, beta=b)               # b A + c A A
            nx = x.clone()
            gemm(B, x, b_mn=True, out=nx, alpha=1.0, beta=a)  # a x + B x
            x = nx
    else:
        for _ in range(steps):
            A = x @ x.transpose(-2, -1)
            B = b * A + c * (A @ A)
            x = a * x + B @ x
    if transposed:
        x = x.transpose(-2, -1)
    return x.to(g.dtype)


def _backend(group) -> str:
    return str(dist.get_backend(group)) if dist.is_initialized() else ""


class _Group:
    """One flat buffer set plus how its gradients are reduced.

    ``reduce_group``  ranks that hold replicas of these parameters (gradients are summed);
    ``norm_group``    ranks over which the parameters are *partitioned* (expert parallelism),
                      whose squared gradient norms add up;
    ``shard_group``   when given, optimizer state is partitioned ZeRO-style over it: the flat
                      gradient is reduce-scattered, every rank updates its 1/N slice of the
                      fp32 master / moments, and the compute-dtype parameters are all-gathered
                      back. The bf16 parameters themselves stay replicated: with 180 GB per
                      GPU there is nothing to gain from re-gathering them layer by layer.
    """

    def __init__(self, kind: str, named_params, reduce_group, norm_group, shard_group=None, p2p: bool = False):
        self.reduce_group, self.norm_group = reduce_group, norm_group
        self.p2p = None
        self.shard_n = dist.get_world_size(shard_group) if (shard_group is not None and dist.is_initialized()) else 1
        self.shard_group = shard_group if self.shard_n > 1 else None
        self.shard_rank = dist.get_rank(shard_group) if self.shard_group is not None else 0
        sharded = self.shard_group is not None
        alloc = None
        if p2p and sharded and self.shard_n <= 8 and any(p.is_cuda for _, p in named_params):
            # flat parameters and gradients in symmetric memory: the two collectives become peer loads / stores
            def alloc(numel, dtype, self=self, named_params=named_params):
                from ..parallel.p2p_zero import P2PShardCollectives

                dev = next(p for _, p in named_params if p.requires_grad).device
                self.p2p = P2PShardCollectives(self.shard_group, numel, dtype, dev)
                return self.p2p.flat, self.p2p.grad
        self.buf = FlatBuffers(named_params, pad_to=8 * self.shard_n, full_master=not sharded, alloc=alloc)
        n, dev = self.buf.numel // self.shard_n, self.buf.device
        self.shard_len = n
        lo = self.shard_rank * n
        self.flat_shard = self.buf.flat[lo:lo + n]
        if sharded:
            self.master = self.flat_shard.float().clone()
            self.grad_shard = torch.zeros(n, dtype=torch.float32, device=dev)
        else:
            self.master = self.buf.master
            self.grad_shard = self.buf.grad
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev) if kind in ("adamw", "sgd", "muon") else None
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev) if kind in ("adamw", "muon") else None
        self.buf.install_hooks()

    @property
    def sharded(self) -> bool:
        return self.shard_group is not None

    @property
    def lowp_out(self):
        """Compute-dtype destination of the update, or None when the master *is* the parameter."""
        if self.sharded:
            return self.flat_shard
        return self.buf.flat if self.buf.has_lowp else None

    def reduce(self) -> None:
        if not dist.is_initialized():
            return
        if self.sharded:
            if self.p2p is not None:
                self.p2p.reduce_scatter(self.grad_shard, self.shard_rank * self.shard_len)
            elif _backend(self.shard_group) == "gloo":
                dist.all_reduce(self.buf.grad, group=self.shard_group)
                lo = self.shard_rank * self.shard_len
                self.grad_shard.copy_(self.buf.grad[lo:lo + self.shard_len])
            else:
                dist.reduce_scatter_tensor(self.grad_shard, self.buf.grad, op=dist.ReduceOp.SUM,
                                           group=self.shard_group)
            if self.reduce_group is not None and dist.get_world_size(self.reduce_group) > 1:
                dist.all_reduce(self.grad_shard, group=self.reduce_group)
        elif self.reduce_group is not None and dist.get_world_size(self.reduce_group) > 1:
            dist.all_reduce(self.buf.grad, op=dist.ReduceOp.SUM, group=self.reduce_group)

    def publish(self) -> None:
        """After the update: make the new parameters visible in the replicated flat buffer."""
        if self.sharded:
            if self.p2p is not None:
                self.p2p.all_gather(self.shard_rank * self.shard_len, self.shard_len)
            elif _backend(self.shard_group) == "gloo":
                parts = [torch.empty_like(self.flat_shard) for _ in range(self.shard_n)]
                dist.all_gather(parts, self.flat_shard.contiguous(), group=self.shard_group)
                self.buf.flat.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(self.buf.flat, self.flat_shard, group=self.shard_group)
        else:
            self.buf.sync_from_master()

    lowp_written_by_kernel = False

    def gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        """Full-length copy of a sharded state tensor (checkpointing)."""
        if not self.sharded:
            return shard
        parts = [torch.empty_like(shard) for _ in range(self.shard_n)]
        dist.all_gather(parts, shard.contiguous(), group=self.shard_group)
        return torch.cat(parts)

    def scatter_full(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        lo = self.shard_rank * self.shard_len
        shard.copy_(full[lo:lo + self.shard_len])


class _FSDPGroup:
    """Optimizer group over parameters that are sharded by ``parallel/fsdp.py``: the rank's persistent slice of
    every unit is the compute-dtype destination of the update, the reduce-scatter already happened unit by unit
    during the backward pass, and nothing is all-gathered after the step (the next forward pulls fresh slices).
    Presents the attributes ``FlatOptimizer`` uses of ``_Group``."""

    p2p = None
    lowp_written_by_kernel = False

    def __init__(self, kind: str, sharded, runtime, reduce_group=None):
        self.buf, self.runtime = sharded, runtime
        self.shard_group, self.shard_n, self.shard_rank = sharded.group, sharded.N, sharded.rank
        self.reduce_group, self.norm_group = reduce_group, None
        n, dev = sharded.shard_numel, sharded.device
        self.shard_len = n
        self.flat_shard = sharded.flat_shard
        self.master = sharded.flat_shard.float().clone()
        self.grad_shard = sharded.grad_shard
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev) if kind in ("adamw", "sgd", "muon") else None
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev) if kind in ("adamw", "muon") else None

    sharded = True

    @property
    def lowp_out(self):
        return self.flat_shard

    def reduce(self) -> None:
        self.runtime.finish_backward()
        if self.reduce_group is not None and dist.get_world_size(self.reduce_group) > 1:
            dist.all_reduce(self.grad_shard, group=self.reduce_group)       # HSDP: sum over the replicas

    def publish(self) -> None:
        self.runtime.after_optimizer_step()

    def gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        return self.buf.gather_full(shard)

    def scatter_full(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        self.buf.scatter_full(full, shard)


class FlatOptimizer:
    """SGD / AdamW / SignSGD / Muon over one or more ``FlatBuffers`` groups (dense parameters
    replicated over the data-parallel ranks, expert parameters sharded over the
    expert-parallel ranks)."""

    def __init__(self, config, named_params, *, max_steps: int | None = None, scheduler_config=None,
                 dp_group=None, expert_params=None, expert_reduce_group=None, expert_norm_group=None,
                 shard_group=None, replicate_group=None, expert_shard_group=None, offload: str | None = None,
                 offload_chunk: int = 16 * 1024 * 1024, p2p_collectives: bool = False, fsdp=None,
                 offload_gradients: bool = False, max_pinned_slots: int | None = None):
        """``fsdp``: ``(ShardedParameters, FSDPRuntime)`` when the dense parameters are sharded (ZeRO-3); the
        dense group then works on the persistent slices and ``named_params`` is ignored. ``offload_gradients``
        (with ``offload = "cpu"`` and ``fsdp``): every layer's reduced gradient slice leaves for host memory as
        soon as its reduce-scatter is done and is accumulated there, under the rest of the backward pass
        (``optim_offload.GradientOffload``)."""
        self.config = config
        self.kind = config.type
        self.step_count = 0
        if self.kind == "muon":
            if fsdp is not None and not getattr(config, "distributed", True):
                raise ValueError("Muon over sharded parameters (model.zero_stage = 3) needs optim.distributed = true")
            if not getattr(config, "distributed", True):
                shard_group = expert_shard_group = None     # every rank keeps whole state and orthogonalises everything
        if fsdp is not None:
            self.groups = [_FSDPGroup(self.kind, fsdp[0], fsdp[1], reduce_group=replicate_group)]
        else:
            self.groups = [_Group(self.kind, named_params, replicate_group if shard_group is not None else dp_group,
                                  None, shard_group, p2p=p2p_collectives)]
        if expert_params and any(p.requires_grad for _, p in expert_params):
            self.groups.append(_Group(self.kind, expert_params,
                                      None if expert_shard_group is not None else expert_reduce_group,
                                      expert_norm_group, expert_shard_group, p2p=p2p_collectives))
        self.schedule = LRSchedule(scheduler_config, max_steps, config.lr) if scheduler_config is not None \
            else LRSchedule(type("C", (), {"type": "constant"})(), max_steps, config.lr)
        dev = self.groups[0].buf.device
        self.hyper = torch.zeros(3, dtype=torch.float32, device=dev)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.last_grad_norm: torch.Tensor | None = None
        # optimizer state in host memory: "state" parks it there between steps, "cpu" also runs the update there
        self.offload = offload
        self._state_offload, self._cpu_step, self._grad_offload = [], [], []
        if offload == "state":
            from .optim_offload import StateOffload

            self._state_offload = [StateOffload(g) for g in self.groups]
        elif offload == "cpu":
            from .optim_offload import CPUStep

            self._cpu_step = [CPUStep(g, self.kind, offload_chunk) for g in self.groups]
            self._grad_offload = [None] * len(self.groups)
            if offload_gradients and fsdp is not None:
                from .optim_offload import GradientOffload

                go = GradientOffload(self.groups[0].shard_len, dev, offload_chunk, max_pinned_slots)
                self._grad_offload[0] = go
                fsdp[0].grad_sink = go.submit_at
        elif offload is not None:
            raise ValueError(f"unknown optimizer offload mode {offload}")

    # ------------------------------------------------------------------ API
    @property
    def buf(self):
        return self.groups[0].buf

    @property
    def lr(self) -> float:
        return self.schedule.lr_at(self.step_count)

    def zero_grad(self) -> None:
        for g in self.groups:
            g.buf.zero_grad()

    def reduce_gradients(self) -> None:
        """Sum each flat gradient over its replica group (one collective per group)."""
        for g in self.groups:
            g.reduce()

    def _global_sumsq(self) -> torch.Tensor:
        self._sumsq.zero_()
        for gi, g in enumerate(self.groups):
            part = torch.zeros_like(self._sumsq)
            go = self._grad_offload[gi] if self._grad_offload else None
            if go is not None:                        # the gradient lives in the host accumulator
                part += float(go.wait().double().pow(2).sum())
            else:
                optim_ops.sumsq(g.grad_shard, part)
            if dist.is_initialized():
                if g.sharded:
                    dist.all_reduce(part, group=g.shard_group)
                if g.norm_group is not None and dist.get_world_size(g.norm_group) > 1:
                    dist.all_reduce(part, group=g.norm_group)
            self._sumsq += part
        return self._sumsq

    def step(self) -> torch.Tensor:
        """Clips, updates and returns the (pre-clip) gradient norm as a device tensor."""
        c = self.config
        lr = self.lr
        self.step_count += 1
        t = self.step_count
        from ..ops import fp8 as fp8_ops

        fp8_ops.bump_weight_epoch()          # fp8 copies of the weights (fp8 training) are stale after this step
        max_norm = c.max_norm if c.max_norm is not None else 0.0
        coef, norm = optim_ops.clip_coef(self._global_sumsq(), max_norm)
        self.last_grad_norm = norm
        if self.kind == "adamw" and self.hyper.is_cuda:
            b1, b2 = c.betas1, c.betas2
            self.hyper.copy_(torch.tensor([lr, 1 - b1 ** t, math.sqrt(1 - b2 ** t)]), non_blocking=True)
        if self._cpu_step:
            scale = float(coef)                       # host value: the update runs on the CPU
            for gi, (g, cs) in enumerate(zip(self.groups, self._cpu_step)):
                go = self._grad_offload[gi]
                # writes the new parameters to the device
                cs.step(lr=lr, grad_scale=scale, t=t, cfg=c, host_grad=go.wait() if go is not None else None)
                if go is not None:
                    go.reset()
                g.lowp_written_by_kernel = True
                if g.sharded:
                    g.publish()
            return norm
        for so in self._state_offload:
            so.load()
        for g in self.groups:
            self._step_group(g, lr, coef, t)
        for so in self._state_offload:
            so.store()
        return norm

    def _step_group(self, g: _Group, lr: float, coef: torch.Tensor, t: int) -> None:
        c, buf = self.config, g.buf
        master, grad = g.master, g.grad_shard
        g.lowp_written_by_kernel = False
        if self.kind == "adamw":
            b1, b2 = c.betas1, c.betas2
            if buf.device.type == "cuda":
                lowp = g.lowp_out
                if lowp is not None and lowp.dtype != torch.bfloat16:
                    lowp = None
                optim_ops.adamw_flat(master, g.exp_avg, g.exp_avg_sq, grad, lowp, self.hyper, b1=b1, b2=b2,
                                     eps=getattr(c, "eps", 1e-8), wd=c.weight_decay, clip=coef)
                g.lowp_written_by_kernel = lowp is not None
            else:
                optim_ops.adamw_ref(master, g.exp_avg, g.exp_avg_sq, grad * coef, lr=lr, b1=b1, b2=b2,
                                    eps=getattr(c, "eps", 1e-8), wd=c.weight_decay, step=t)
        elif self.kind == "sgd":
            gr = grad * coef
            if c.weight_decay:
                gr = gr + c.weight_decay * master
            g.exp_avg.mul_(c.momentum).add_(gr)
            upd = gr + c.momentum * g.exp_avg if c.nesterov else g.exp_avg
            master.add_(upd, alpha=-lr)
        elif self.kind == "sign_sgd":
            gr = grad * coef
            master.mul_(1 - lr * c.weight_decay).add_(torch.sign(gr), alpha=-lr)
        elif self.kind == "muon":
            self._muon_step(g, lr, coef, t)
        else:
            raise ValueError(f"unknown optimizer {self.kind}")
        if g.sharded and not g.lowp_written_by_kernel:
            g.flat_shard.copy_(master)
            g.lowp_written_by_kernel = True
        g.publish()

    def _muon_step(self, grp: _Group, lr: float, coef: torch.Tensor, t: int) -> None:
        """Muon on >= 2-D matrices that are not embeddings / heads; AdamW on the rest
        (the split the reference makes, trainer/optim/__init__.py:151-249)."""
        c, buf = self.config, grp.buf
        if grp.sharded:
            return self._muon_step_sharded(grp, lr, coef, t)
        g_all = buf.grad * coef
        b1, b2 = c.betas1, c.betas2
        is_matrix = self._is_muon_matrix

        # The gradients are identical on the ranks of the reduction group, so the orthogonalisations can be dealt
        # out: every matrix has one owner (largest first onto the least loaded rank), which writes its scaled update
        # into a buffer that is zero elsewhere; one sum over the ranks hands every update to everybody. The reference
        # moves whole matrices to their owners with an all-to-all and gathers the updates
        # (trainer/optim/__init__.py:151-249); with replicated gradients only the second half is needed.
        group = grp.reduce_group
        world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        owner: dict[str, int] = {}
        shared_upd = None
        if getattr(c, "distributed", True) and world > 1:
            rank = dist.get_rank(group)
            load = [0.0] * world
            mats = sorted((s for s in buf.slots if is_matrix(s)), key=lambda s: (-s.numel * min(s.shape[-2:]), s.name))
            for s in mats:
                r = min(range(world), key=lambda i: (load[i], i))
                owner[s.name] = r
                load[r] += s.numel * min(s.shape[-2:])
            shared_upd = torch.zeros_like(buf.master)
        for s in buf.slots:
            sl = slice(s.offset, s.offset + s.numel)
            g = g_all[sl].view(s.shape)
            p = buf.master[sl].view(s.shape)
            m = grp.exp_avg[sl].view(s.shape)
            if is_matrix(s):
                m.mul_(c.mu).add_(g)
                rows, cols = s.shape[-2], s.shape[-1]
                scale = 0.2 * math.sqrt(max(rows, cols)) if c.adjust_lr == "rms_norm" else \
                    (math.sqrt(max(1.0, rows / cols)) if c.adjust_lr == "spectral_norm" else 1.0)
                if shared_upd is not None:
                    if owner[s.name] == rank:
                        shared_upd[sl].view(s.shape).copy_(newton_schulz(g + c.mu * m, c.ns_steps).float() * scale)
                    continue
                upd = newton_schulz(g + c.mu * m, c.ns_steps).float()
                p.mul_(1 - lr * c.weight_decay).add_(upd, alpha=-lr * scale)
            else:
                v = grp.exp_avg_sq[sl].view(s.shape)
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = v.sqrt() / math.sqrt(1 - b2 ** t) + 1e-8
                p.mul_(1 - lr * c.weight_decay).addcdiv_(m, denom, value=-lr / (1 - b1 ** t))
        if shared_upd is not None:
            dist.all_reduce(shared_upd, group=group)
            self.muon_owned = sum(1 for r in owner.values() if r == rank)
            for s in buf.slots:
                if s.name in owner:
                    sl = slice(s.offset, s.offset + s.numel)
                    buf.master[sl].mul_(1 - lr * c.weight_decay).add_(shared_upd[sl], alpha=-lr)

    @staticmethod
    def _is_muon_matrix(s) -> bool:
        return len(s.shape) >= 2 and "embed" not in s.name and "lm_head" not in s.name

    @staticmethod
    def _muon_scale(c, shape) -> float:
        rows, cols = shape[-2], shape[-1]
        if c.adjust_lr == "rms_norm":
            return 0.2 * math.sqrt(max(rows, cols))
        return math.sqrt(max(1.0, rows / cols)) if c.adjust_lr == "spectral_norm" else 1.0

    def _muon_step_sharded(self, grp: _Group, lr: float, coef: torch.Tensor, t: int) -> None:
        """Muon over an optimizer group whose state is partitioned (ZeRO-2): master weights, momentum and the reduced
        gradient exist as one flat slice per rank, and matrices straddle the slices. Momentum and the Nesterov
        direction are elementwise on the slice; the directions are all-gathered so that the owner of every matrix
        (dealt out by cost) can orthogonalise it whole; the scaled updates come back through a reduce-scatter of a buffer
        that is zero outside the owned matrices. Elements outside the Muon matrices take an AdamW step on the slice.
        (The reference moves matrix shards to their owners and back with all-to-alls, trainer/optim/__init__.py:151-249;
        the two collectives here carry the whole flat buffer, transiently 8 bytes per parameter.)"""
        c, buf = self.config, grp.buf
        n, lo = grp.shard_len, grp.shard_rank * grp.shard_len
        world, rank = grp.shard_n, grp.shard_rank
        dev = grp.master.device
        by_unit = isinstance(grp, _FSDPGroup)         # ZeRO-3: the rank's slice is one piece per layer unit

        def my_slice(full: torch.Tensor) -> torch.Tensor:
            if not by_unit:
                return full[lo:lo + n].clone()
            out = torch.empty(n, dtype=full.dtype, device=dev)
            buf.scatter_full(full, out)
            return out

        mask = getattr(grp, "_muon_mask", None)
        if mask is None:
            full = torch.zeros(buf.numel, dtype=torch.float32, device=dev)
            for s in buf.slots:
                if self._is_muon_matrix(s):
                    full[s.offset:s.offset + s.numel] = 1.0
            mask = grp._muon_mask = my_slice(full) > 0
        g = grp.grad_shard * coef
        m, v, p = grp.exp_avg, grp.exp_avg_sq, grp.master
        b1, b2 = c.betas1, c.betas2
        # elementwise part on the slice: Muon momentum inside the matrices, AdamW outside
        m_muon = m * c.mu + g
        m_adam = m * b1 + g * (1 - b1)
        m.copy_(torch.where(mask, m_muon, m_adam))
        v.copy_(torch.where(mask, v, v * b2 + g * g * (1 - b2)))
        direction = torch.where(mask, g + c.mu * m, torch.zeros_like(g))
        full_dir = grp.gather_full(direction)
        upd = torch.zeros_like(full_dir)
        load = [0.0] * world
        mats = sorted((s for s in buf.slots if self._is_muon_matrix(s)), key=lambda s: (-s.numel * min(s.shape[-2:]), s.name))
        owned = 0
        for s in mats:
            r = min(range(world), key=lambda i: (load[i], i))
            load[r] += s.numel * min(s.shape[-2:])
            if r == rank:
                sl = slice(s.offset, s.offset + s.numel)
                upd[sl].view(s.shape).copy_(newton_schulz(full_dir[sl].view(s.shape), c.ns_steps).float()
                                            * self._muon_scale(c, s.shape))
                owned += 1
        self.muon_owned = owned
        if by_unit or _backend(grp.shard_group) == "gloo":
            dist.all_reduce(upd, group=grp.shard_group)
            mine = my_slice(upd)
        else:
            mine = torch.empty(n, dtype=upd.dtype, device=dev)
            dist.reduce_scatter_tensor(mine, upd, op=dist.ReduceOp.SUM, group=grp.shard_group)
        denom = v.sqrt() / math.sqrt(1 - b2 ** t) + 1e-8
        adam = m / denom / (1 - b1 ** t)
        p.mul_(1 - lr * c.weight_decay).add_(torch.where(mask, mine, adam), alpha=-lr)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        """Per-parameter (name-keyed) tensors, so that a checkpoint does not depend on the
        flat layout."""
        out: dict = {"step": self.step_count, "state": {}}
        for g in self.groups:
            for key, flat in (("master", g.master), ("exp_avg", g.exp_avg), ("exp_avg_sq", g.exp_avg_sq)):
                if flat is not None:
                    out["state"].setdefault(key, {}).update(g.buf.named_views(g.gather_full(flat)))
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for g in self.groups:
            for key, flat in (("master", g.master), ("exp_avg", g.exp_avg), ("exp_avg_sq", g.exp_avg_sq)):
                if flat is None or key not in sd.get("state", {}):
                    continue
                full = g.gather_full(flat).clone() if g.sharded else flat
                views = g.buf.named_views(full)
                for name, t in sd["state"][key].items():
                    if name in views:
                        views[name].copy_(t)
                if g.sharded:
                    g.scatter_full(full, flat)
        self.sync_from_master()

    def sync_from_master(self) -> None:
        """Re-derive the compute-dtype parameters from the fp32 master copy."""
        for g in self.groups:
            if g.sharded:
                g.flat_shard.copy_(g.master)
                g.lowp_written_by_kernel = True
                g.publish()
            else:
                g.buf.sync_from_master()


def setup_optimizer(config, model, *, max_steps=None, scheduler_config=None, dp_group=None,
                    expert_reduce_group=None, expert_norm_group=None, shard_group=None, replicate_group=None,
                    expert_shard_group=None, offload: str | None = None,
                    offload_chunk: int = 16 * 1024 * 1024, p2p_collectives: bool = False, fsdp=None,
                    offload_gradients: bool = False, max_pinned_slots: int | None = None) -> FlatOptimizer:
    """Parameters marked ``_is_expert_shard`` (set by the expert-parallel setup) form their own
    group: they are reduced over the ranks that replicate the same expert shard."""
    dense = [(n, p) for n, p in model.named_parameters() if not getattr(p, "_is_expert_shard", False)]
    expert = [(n, p) for n, p in model.named_parameters() if getattr(p, "_is_expert_shard", False)]
    return FlatOptimizer(config, dense, max_steps=max_steps, scheduler_config=scheduler_config, dp_group=dp_group,
                         expert_params=expert, expert_reduce_group=expert_reduce_group,
                         expert_norm_group=expert_norm_group, shard_group=shard_group,
                         replicate_group=replicate_group, expert_shard_group=expert_shard_group, offload=offload,
                         offload_chunk=offload_chunk, p2p_collectives=p2p_collectives, fsdp=fsdp,
                         offload_gradients=offload_gradients, max_pinned_slots=max_pinned_slots)
