"""Optimizer-state placement in host memory for the flat-buffer optimizer.

``state``  (``model.optim_cpu_offload``): fp32 master weights and moments rest in pinned host
           memory and visit the GPU only around ``step()`` (the reference's
           ``CPUOffloadOptimizer``, src/prime_rl/trainer/optim/state_offload.py).
``cpu``    (``model.full_offload``): the update itself runs on the CPU with the vectorised C++
           optimizer (``csrc/cpu/cpu_optim.cpp``). The flat gradient shard is streamed to pinned
           host memory in chunks, each chunk is updated while the next one is in flight, and the
           new compute-dtype parameters are streamed back (the reference's
           ``FullCPUOffloadOptimizer``, trainer/optim/offload.py:1058-1375, same 16 Mi-element
           chunking).
"""

from __future__ import annotations

import torch

from ..ops import cpu_optim

STATE_NAMES = ("master", "exp_avg", "exp_avg_sq")


def _pinned_like(t: torch.Tensor, pin: bool) -> torch.Tensor:
    out = torch.empty(t.shape, dtype=t.dtype, device="cpu")
    if pin and torch.cuda.is_available():
        out = out.pin_memory()
    return out


class StateOffload:
    """Keeps a group's separate state tensors on the host between steps."""

    def __init__(self, group):
        self.group = group
        self.dev = group.buf.device
        self.host: dict[str, torch.Tensor] = {}
        for name in STATE_NAMES:
            t = getattr(group, name)
            # a master that *is* the parameter buffer (fp32 training, unsharded) has to stay
            if t is None or (name == "master" and t is group.buf.flat):
                continue
            h = _pinned_like(t, self.dev.type == "cuda")
            h.copy_(t)
            self.host[name] = h
            setattr(group, name, h)

    def load(self) -> None:
        for name, h in self.host.items():
            setattr(self.group, name, h.to(self.dev, non_blocking=True))

    def store(self) -> None:
        for name, h in self.host.items():
            h.copy_(getattr(self.group, name), non_blocking=True)
            setattr(self.group, name, h)
        if self.dev.type == "cuda":
            torch.cuda.current_stream(self.dev).synchronize()


class CPUStep:
    """AdamW / SignSGD of one group on the host, chunk-pipelined with the transfers."""

    def __init__(self, group, kind: str, chunk_elements: int = 16 * 1024 * 1024):
        if kind not in ("adamw", "sign_sgd"):
            raise ValueError(f"the CPU optimizer supports adamw and sign_sgd, not {kind}")
        self.group, self.kind, self.chunk = group, kind, int(chunk_elements)
        self.dev = group.buf.device
        cuda = self.dev.type == "cuda"
        n = group.shard_len
        self.master = group.master.detach().float().cpu().contiguous()
        self.exp_avg = torch.zeros(n, dtype=torch.float32) if kind == "adamw" else None
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32) if kind == "adamw" else None
        # device destination of the new parameters (taken before the group's state moves to the host)
        self.dest = group.lowp_out if group.lowp_out is not None else group.master
        # the group's state now lives on the host (checkpointing reads it through the group)
        group.master, group.exp_avg, group.exp_avg_sq = self.master, self.exp_avg, self.exp_avg_sq
        c = min(self.chunk, n)
        out_dtype = self.dest.dtype
        self.grad_slots = [_pinned_like(torch.empty(c, dtype=group.grad_shard.dtype), cuda) for _ in range(2)]
        self.out_slots = [_pinned_like(torch.empty(c, dtype=out_dtype), cuda) for _ in range(2)]
        self.stream = torch.cuda.Stream(device=self.dev) if cuda else None

    def step(self, *, lr: float, grad_scale: float, t: int, cfg) -> None:
        g, n, C = self.group, self.group.shard_len, self.chunk
        dest = self.dest
        chunks = [(lo, min(lo + C, n)) for lo in range(0, n, C)]
        cuda = self.stream is not None
        if cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.dev))
        d2h = [None] * len(chunks)
        h2d_done: list = [None, None]

        def fetch(i):
            lo, hi = chunks[i]
            slot = self.grad_slots[i & 1][: hi - lo]
            if cuda:
                with torch.cuda.stream(self.stream):
                    slot.copy_(g.grad_shard[lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                d2h[i] = ev
            else:
                slot.copy_(g.grad_shard[lo:hi])

        fetch(0)
        for i, (lo, hi) in enumerate(chunks):
            if cuda:
                d2h[i].synchronize()
            if i + 1 < len(chunks):
                fetch(i + 1)
            if cuda and h2d_done[i & 1] is not None:
                h2d_done[i & 1].synchronize()          # the out slot is free again
            grad = self.grad_slots[i & 1][: hi - lo]
            out = self.out_slots[i & 1][: hi - lo]
            if self.kind == "adamw":
                cpu_optim.cpu_adamw_step(self.master[lo:hi], self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], grad, out,
                                         step=t, lr=lr, b1=cfg.betas1, b2=cfg.betas2, eps=getattr(cfg, "eps", 1e-8),
                                         wd=cfg.weight_decay, grad_scale=grad_scale)
            else:
                cpu_optim.cpu_sign_sgd_step(self.master[lo:hi], grad, out, lr=lr, wd=cfg.weight_decay,
                                            grad_scale=grad_scale)
            if cuda:
                with torch.cuda.stream(self.stream):
                    dest[lo:hi].copy_(out, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                h2d_done[i & 1] = ev
            else:
                dest[lo:hi].copy_(out)
        if cuda:
            torch.cuda.current_stream(self.dev).wait_stream(self.stream)

    def state(self) -> dict:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}
