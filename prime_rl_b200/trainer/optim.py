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
                 align: int = 8):
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
        self.numel = off
        self.params = [p for _, p in params]
        self.flat = torch.zeros(off, dtype=self.dtype, device=self.device)
        for s, p in zip(self.slots, self.params):
            view = self.flat[s.offset:s.offset + s.numel].view(s.shape)
            view.copy_(p.data)
            p.data = view
        if self.dtype == master_dtype:
            self.master = self.flat
        else:
            self.master = self.flat.to(master_dtype)
        self.grad = torch.zeros(off, dtype=torch.float32, device=self.device)
        self._grad_views = [self.grad[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots]

    @property
    def has_lowp(self) -> bool:
        return self.master is not self.flat

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
                gv.add_(param.grad)
                param.grad = None
            p.register_post_accumulate_grad_hook(hook)

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
    """Quintic Newton-Schulz orthogonalisation used by Muon (bf16 on GPU)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.to(torch.bfloat16 if g.is_cuda else torch.float32)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-2, -1)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = x @ x.transpose(-2, -1)
        B = b * A + c * (A @ A)
        x = a * x + B @ x
    if transposed:
        x = x.transpose(-2, -1)
    return x.to(g.dtype)


class FlatOptimizer:
    """SGD / AdamW / SignSGD / Muon over ``FlatBuffers``."""

    def __init__(self, config, named_params, *, max_steps: int | None = None, scheduler_config=None,
                 dp_group=None, grad_divide: float = 1.0):
        self.config = config
        self.buf = FlatBuffers(named_params)
        self.kind = config.type
        self.step_count = 0
        self.dp_group = dp_group
        self.grad_divide = grad_divide
        self.schedule = LRSchedule(scheduler_config, max_steps, config.lr) if scheduler_config is not None \
            else LRSchedule(type("C", (), {"type": "constant"})(), max_steps, config.lr)
        n, dev = self.buf.numel, self.buf.device
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev) if self.kind in ("adamw", "sgd", "muon") else None
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev) if self.kind in ("adamw", "muon") else None
        self.hyper = torch.zeros(3, dtype=torch.float32, device=dev)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.last_grad_norm: torch.Tensor | None = None
        self.buf.install_hooks()

    # ------------------------------------------------------------------ API
    @property
    def lr(self) -> float:
        return self.schedule.lr_at(self.step_count)

    def zero_grad(self) -> None:
        self.buf.zero_grad()

    def reduce_gradients(self) -> None:
        """Sum the flat gradient over the data-parallel group (one collective)."""
        if self.dp_group is not None and dist.is_initialized() and dist.get_world_size(self.dp_group) > 1:
            dist.all_reduce(self.buf.grad, op=dist.ReduceOp.SUM, group=self.dp_group)

    def step(self) -> torch.Tensor:
        """Clips, updates and returns the (pre-clip) gradient norm as a device tensor."""
        c, buf = self.config, self.buf
        lr = self.lr
        self.step_count += 1
        t = self.step_count
        max_norm = c.max_norm if c.max_norm is not None else 0.0
        self._sumsq.zero_()
        optim_ops.sumsq(buf.grad, self._sumsq)
        coef, norm = optim_ops.clip_coef(self._sumsq, max_norm)
        self.last_grad_norm = norm
        if self.kind == "adamw":
            b1, b2 = c.betas1, c.betas2
            if buf.device.type == "cuda":
                self.hyper.copy_(torch.tensor([lr, 1 - b1 ** t, math.sqrt(1 - b2 ** t)]), non_blocking=True)
                optim_ops.adamw_flat(buf.master, self.exp_avg, self.exp_avg_sq, buf.grad,
                                     buf.flat if buf.has_lowp else None, self.hyper, b1=b1, b2=b2,
                                     eps=getattr(c, "eps", 1e-8), wd=c.weight_decay, clip=coef)
            else:
                optim_ops.adamw_ref(buf.master, self.exp_avg, self.exp_avg_sq, buf.grad * coef, lr=lr, b1=b1, b2=b2,
                                    eps=getattr(c, "eps", 1e-8), wd=c.weight_decay, step=t)
                buf.sync_from_master()
        elif self.kind == "sgd":
            g = buf.grad * coef
            if c.weight_decay:
                g = g + c.weight_decay * buf.master
            self.exp_avg.mul_(c.momentum).add_(g)
            upd = g + c.momentum * self.exp_avg if c.nesterov else self.exp_avg
            buf.master.add_(upd, alpha=-lr)
            buf.sync_from_master()
        elif self.kind == "sign_sgd":
            g = buf.grad * coef
            buf.master.mul_(1 - lr * c.weight_decay).add_(torch.sign(g), alpha=-lr)
            buf.sync_from_master()
        elif self.kind == "muon":
            self._muon_step(lr, coef, t)
        else:
            raise ValueError(f"unknown optimizer {self.kind}")
        return norm

    def _muon_step(self, lr: float, coef: torch.Tensor, t: int) -> None:
        """Muon on >= 2-D matrices that are not embeddings / heads; AdamW on the rest
        (the split the reference makes, trainer/optim/__init__.py:151-249)."""
        c, buf = self.config, self.buf
        g_all = buf.grad * coef
        b1, b2 = c.betas1, c.betas2
        for s in buf.slots:
            sl = slice(s.offset, s.offset + s.numel)
            g = g_all[sl].view(s.shape)
            p = buf.master[sl].view(s.shape)
            m = self.exp_avg[sl].view(s.shape)
            is_matrix = len(s.shape) >= 2 and "embed" not in s.name and "lm_head" not in s.name
            if is_matrix:
                m.mul_(c.mu).add_(g)
                upd = newton_schulz(g + c.mu * m, c.ns_steps).float()
                rows, cols = s.shape[-2], s.shape[-1]
                scale = 0.2 * math.sqrt(max(rows, cols)) if c.adjust_lr == "rms_norm" else \
                    (math.sqrt(max(1.0, rows / cols)) if c.adjust_lr == "spectral_norm" else 1.0)
                p.mul_(1 - lr * c.weight_decay).add_(upd, alpha=-lr * scale)
            else:
                v = self.exp_avg_sq[sl].view(s.shape)
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = v.sqrt() / math.sqrt(1 - b2 ** t) + 1e-8
                p.mul_(1 - lr * c.weight_decay).addcdiv_(m, denom, value=-lr / (1 - b1 ** t))
        buf.sync_from_master()

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        """Per-parameter (name-keyed) tensors, so that a checkpoint does not depend on the
        flat layout."""
        out: dict = {"step": self.step_count, "state": {}}
        for key, flat in (("master", self.buf.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            if flat is not None:
                out["state"][key] = self.buf.named_views(flat)
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for key, flat in (("master", self.buf.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            if flat is None or key not in sd.get("state", {}):
                continue
            views = self.buf.named_views(flat)
            for name, t in sd["state"][key].items():
                if name in views:
                    views[name].copy_(t)
        self.buf.sync_from_master()


def setup_optimizer(config, model, *, max_steps=None, scheduler_config=None, dp_group=None) -> FlatOptimizer:
    return FlatOptimizer(config, list(model.named_parameters()), max_steps=max_steps,
                         scheduler_config=scheduler_config, dp_group=dp_group)
