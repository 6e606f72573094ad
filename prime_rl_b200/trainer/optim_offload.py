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

    def step(self, *, lr: float, grad_scale: float, t: int, cfg, host_grad: torch.Tensor | None = None) -> None:
        """``host_grad``: the complete fp32 gradient shard already in host memory (``GradientOffload``): nothing
        is fetched from the device, only the new parameters travel."""
        g, n, C = self.group, self.group.shard_len, self.chunk
        dest = self.dest
        chunks = [(lo, min(lo + C, n)) for lo in range(0, n, C)]
        cuda = self.stream is not None
        if cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.dev))
        d2h = [None] * len(chunks)
        h2d_done: list = [None, None]

        def fetch(i):
            if host_grad is not None:
                return
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
            if cuda and host_grad is None:
                d2h[i].synchronize()
            if i + 1 < len(chunks):
                fetch(i + 1)
            if cuda and h2d_done[i & 1] is not None:
                h2d_done[i & 1].synchronize()          # the out slot is free again
            grad = self.grad_slots[i & 1][: hi - lo] if host_grad is None else host_grad[lo:hi]
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


class GradientOffload:
    """Gradient accumulation in host memory while the backward pass goes on (the reference's
    ``GradientOffloadManager``, src/prime_rl/trainer/optim/offload.py:93-473).

    ``submit(view)`` is called when a piece of the flat gradient shard is final for the current micro-batch (by
    the optimizer after a micro-batch, or per layer from the parameter-sharding runtime's reduce-scatter hook):
    the piece is copied device -> host on a side stream into one of ``max_pinned_slots`` pinned buffers, the
    device memory is zeroed for the next micro-batch, and a worker thread adds the buffer into the fp32 host
    accumulator (vectorised C++ for bf16 sources) as soon as the copy's event has fired. At most
    ``max_pinned_slots`` pieces are in flight: ``submit`` blocks on the oldest one when all slots are taken, which
    bounds the pinned memory. ``wait()`` returns the accumulator once everything submitted has been added; the
    CPU optimizer step then reads it in place, so the device-to-host copy of the whole shard at step time is gone
    and the transfer rides under the backward pass instead."""

    def __init__(self, shard_len: int, device: torch.device, chunk_elements: int = 16 * 1024 * 1024,
                 max_pinned_slots: int | None = None, src_dtype: torch.dtype = torch.float32):
        import queue
        import threading

        self.n, self.dev, self.chunk = int(shard_len), device, int(min(chunk_elements, max(shard_len, 1)))
        self.cuda = device.type == "cuda"
        self.acc = torch.zeros(self.n, dtype=torch.float32)
        slots = max_pinned_slots or 4
        self.free: "queue.Queue[torch.Tensor]" = queue.Queue()
        for _ in range(slots):
            self.free.put(_pinned_like(torch.empty(self.chunk, dtype=src_dtype), self.cuda))
        self.work: "queue.Queue" = queue.Queue()
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None
        self.error: BaseException | None = None
        self.submitted = 0
        self.stats = {"pieces": 0, "bytes": 0, "slot_waits": 0}
        self._thread = threading.Thread(target=self._worker, name="grad-offload", daemon=True)
        self._thread.start()

    def _worker(self):
        while True:
            item = self.work.get()
            if item is None:
                self.work.task_done()
                return
            slot, lo, hi, event = item
            try:
                if event is not None:
                    event.synchronize()
                src = slot[: hi - lo]
                if src.dtype == torch.bfloat16:
                    cpu_optim.bf16_to_fp32_(self.acc[lo:hi], src, accumulate=True)
                else:
                    self.acc[lo:hi].add_(src)
            except BaseException as e:          # surfaced by wait()
                self.error = e
            finally:
                self.free.put(slot)
                self.work.task_done()

    def submit(self, grad: torch.Tensor, offset: int = 0, zero: bool = True) -> None:
        """``grad``: a contiguous 1-D view of the device gradient shard that starts at element ``offset``."""
        import queue

        n = grad.numel()
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.dev))
        for lo in range(0, n, self.chunk):
            hi = min(lo + self.chunk, n)
            try:
                slot = self.free.get_nowait()
            except queue.Empty:
                self.stats["slot_waits"] += 1
                slot = self.free.get()           # back-pressure: the oldest piece has to land first
            piece = grad[lo:hi]
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    slot[: hi - lo].copy_(piece, non_blocking=True)
                    if zero:
                        piece.zero_()
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                piece.record_stream(self.stream)
            else:
                slot[: hi - lo].copy_(piece)
                if zero:
                    piece.zero_()
                ev = None
            self.work.put((slot, offset + lo, offset + hi, ev))
            self.stats["pieces"] += 1
            self.stats["bytes"] += (hi - lo) * piece.element_size()
        if self.cuda and zero:
            torch.cuda.current_stream(self.dev).wait_stream(self.stream)   # later kernels see the zeroed buffer
        self.submitted += 1

    def submit_at(self, offset: int, grad: torch.Tensor) -> None:
        """Sink signature of the parameter-sharding runtime: a freshly reduced slice, not kept on the device."""
        self.submit(grad, offset, zero=False)

    def wait(self) -> torch.Tensor:
        self.work.join()
        if self.error is not None:
            e, self.error = self.error, None
            raise RuntimeError("gradient offload worker failed") from e
        return self.acc

    def reset(self) -> None:
        self.wait()
        self.acc.zero_()
        self.submitted = 0

    def close(self) -> None:
        self.work.put(None)
        self._thread.join(timeout=10)


def pci_address(device: torch.device) -> str:
    p = torch.cuda.get_device_properties(device)
    return f"{getattr(p, 'pci_domain_id', 0):04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"


def numa_node_of_gpu(pci_bus_id: str, sysfs: str = "/sys") -> int | None:
    """NUMA node the GPU hangs off (``<sysfs>/bus/pci/devices/<id>/numa_node``), None when the platform does not
    say (file missing or -1)."""
    from pathlib import Path

    bus = pci_bus_id.lower()
    if bus.count(":") == 2 and len(bus.split(":")[0]) == 8:      # CUDA prints an 8-digit domain, sysfs uses 4
        bus = bus[4:]
    f = Path(sysfs) / "bus" / "pci" / "devices" / bus / "numa_node"
    try:
        node = int(f.read_text().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def cpus_of_numa_node(node: int, sysfs: str = "/sys") -> set[int]:
    from pathlib import Path

    try:
        text = (Path(sysfs) / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text().strip()
    except OSError:
        return set()
    cpus: set[int] = set()
    for part in filter(None, text.split(",")):
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys", setaffinity=None) -> int | None:
    """Pins this process (and the threads it starts afterwards: the CPU optimizer's workers, the gradient-offload
    thread) to the cores of the GPU's NUMA node, so that pinned buffers are allocated and touched next to the PCIe
    root the copies go through (reference: src/prime_rl/trainer/utils.py:119-170). Returns the node, or None when
    nothing was changed."""
    import os

    node = numa_node_of_gpu(pci_bus_id, sysfs)
    if node is None:
        return None
    cpus = cpus_of_numa_node(node, sysfs)
    allowed = cpus & set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else cpus
    if not allowed:
        return None
    (setaffinity or os.sched_setaffinity)(0, allowed)
    return node
