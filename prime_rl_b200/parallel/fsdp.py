"""Parameter sharding (ZeRO-3 / FSDP): every rank keeps 1 / N of every decoder layer's parameters, of their
fp32 master copy, moments and gradient accumulator; a layer's full bf16 parameters exist only while that
layer runs.

Layout. The trainable parameters of one decoder layer form a *unit*: they are laid out back to back in a flat
range whose length is padded to a multiple of ``N * 8`` elements, and rank r owns the r-th slice of that
range. A rank's persistent storage (``flat_shard``, and the optimizer's master / moments / ``grad_shard`` next
to it) is the concatenation of its slices of all units. Embedding, final norm and LM head form the *root*
unit, which stays gathered for the whole step (both ends of the model use it) and is refreshed after the
optimizer step.

Step. ``CausalLM`` calls ``run(layer, idx, h, seq)`` for every layer, in the forward pass and again when a
checkpointed layer is recomputed in the backward pass. ``run`` makes the unit's parameters views of one of
a small pool of full-size gather buffers (all-gather of the N slices, prefetched for the next unit on a
side stream while the current one computes), so at most ``pool`` units are ever whole. Gradients land, through
per-parameter hooks, in a pooled fp32 unit buffer; when every parameter of the unit has reported, the buffer
is reduce-scattered and the rank's slice is added to ``grad_shard``. The optimizer then updates the shard in
place (``trainer/optim.py``); nothing is all-gathered after the step: the next forward pulls fresh slices.

The two collectives are ``torch.distributed`` calls (NCCL on GPUs, where NVSwitch reduces inside the fabric;
gloo on CPU), issued per unit so that each moves tens to hundreds of MB. Same role as FSDP2's per-block
``fully_shard`` with explicit forward / backward prefetch in the reference
(src/prime_rl/trainer/model.py:470-620).
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class _Slot:
    name: str
    offset: int            # inside the unit's flat range
    numel: int
    shape: torch.Size


@dataclass
class Unit:
    index: int             # decoder layer index, or -1 for the root unit
    params: list[torch.nn.Parameter]
    slots: list[_Slot]
    numel: int             # padded: a multiple of N * align
    shard_offset: int = 0  # where this unit's slice starts inside the rank's persistent shard
    resident: bool = False # root unit: never released
    # runtime state
    buffer: int = -1       # pool buffer that currently holds the gathered parameters
    grad_buffer: int = -1
    pending: int = 0       # parameters that still have to report a gradient in this backward pass
    ready: torch.cuda.Event | None = None


class ShardedParameters:
    """Owns the persistent shards and plays the part of ``FlatBuffers`` for the optimizer group."""

    def __init__(self, units_named: list[tuple[int, list[tuple[str, torch.nn.Parameter]]]], group, *, align: int = 8):
        self.group = group
        self.N = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        first = next(p for _, named in units_named for _, p in named)
        self.device, self.dtype = first.device, first.dtype
        self.units: list[Unit] = []
        off = 0
        for index, named in units_named:
            named = [(n, p) for n, p in named if p.requires_grad]
            if not named:
                continue
            slots, cur = [], 0
            for n, p in named:
                if p.dtype != self.dtype:
                    raise ValueError(f"mixed parameter dtypes ({n}: {p.dtype} vs {self.dtype})")
                slots.append(_Slot(n, cur, p.numel(), p.shape))
                cur += (p.numel() + align - 1) // align * align
            quantum = self.N * align
            numel = (cur + quantum - 1) // quantum * quantum
            u = Unit(index, [p for _, p in named], slots, numel, shard_offset=off, resident=index < 0)
            self.units.append(u)
            off += numel // self.N
        self.shard_numel = off
        self.numel = sum(u.numel for u in self.units)              # length of the (virtual) full flat buffer
        self.flat_shard = torch.zeros(off, dtype=self.dtype, device=self.device)
        self.grad_shard = torch.zeros(off, dtype=torch.float32, device=self.device)
        self.params = [p for u in self.units for p in u.params]
        # full-flat slots (unit-major), for name-keyed checkpoints of gathered optimizer state
        self.slots = []
        base = 0
        for u in self.units:
            for s in u.slots:
                self.slots.append(_Slot(s.name, base + s.offset, s.numel, s.shape))
            base += u.numel
        # keep this rank's slice of the initial values, then let go of the full tensors
        with torch.no_grad():
            for u in self.units:
                full = torch.zeros(u.numel, dtype=self.dtype, device=self.device)
                for s, p in zip(u.slots, u.params):
                    full[s.offset:s.offset + s.numel].copy_(p.data.reshape(-1))
                n = u.numel // self.N
                self.unit_shard(u).copy_(full[self.rank * n:(self.rank + 1) * n])
                for p in u.params:
                    p.data = torch.empty(0, dtype=self.dtype, device=self.device)

    def unit_shard(self, u: Unit, of: torch.Tensor | None = None) -> torch.Tensor:
        t = self.flat_shard if of is None else of
        n = u.numel // self.N
        return t[u.shard_offset:u.shard_offset + n]

    # ---- the FlatBuffers interface the optimizer uses
    def zero_grad(self) -> None:
        self.grad_shard.zero_()
        for p in self.params:
            p.grad = None

    def named_views(self, full_flat: torch.Tensor) -> dict[str, torch.Tensor]:
        return {s.name: full_flat[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots}

    def gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        """Full-length (unit-major) copy of a tensor laid out like the persistent shard."""
        out = torch.empty(self.numel, dtype=shard.dtype, device=shard.device)
        base = 0
        for u in self.units:
            _all_gather(out[base:base + u.numel], self.unit_shard(u, shard), self.group, self.N)
            base += u.numel
        return out

    def scatter_full(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        base = 0
        for u in self.units:
            n = u.numel // self.N
            self.unit_shard(u, shard).copy_(full[base + self.rank * n:base + (self.rank + 1) * n])
            base += u.numel


def _all_gather(out: torch.Tensor, mine: torch.Tensor, group, N: int) -> None:
    if N == 1:
        out.copy_(mine)
    elif str(dist.get_backend(group)) == "gloo":
        parts = list(out.chunk(N))
        dist.all_gather(parts, mine.contiguous(), group=group)
    else:
        dist.all_gather_into_tensor(out, mine.contiguous(), group=group)


def _reduce_scatter(out: torch.Tensor, full: torch.Tensor, group, N: int) -> None:
    if N == 1:
        out.copy_(full)
    elif str(dist.get_backend(group)) == "gloo":
        dist.all_reduce(full, group=group)
        r = dist.get_rank(group)
        out.copy_(full.chunk(N)[r])
    else:
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group)


class FSDPRuntime:
    """Installed as ``CausalLM.layer_hooks``. ``pool``: number of gather buffers (>= 2 for prefetch)."""

    def __init__(self, model, sharded: ShardedParameters, *, pool: int = 2, prefetch: bool = True):
        self.model, self.sp = model, sharded
        self.layer_units = {u.index: u for u in sharded.units if u.index >= 0}
        self.root = next((u for u in sharded.units if u.index < 0), None)
        dev, dt = sharded.device, sharded.dtype
        biggest = max((u.numel for u in self.layer_units.values()), default=0)
        self.keep_all = False          # without recomputation every unit must stay whole until its backward
        self.pool_size = max(2, pool)
        self.param_pool = [torch.empty(biggest, dtype=dt, device=dev) for _ in range(self.pool_size)]
        self.grad_pool = [torch.zeros(biggest, dtype=torch.float32, device=dev) for _ in range(2)]
        self.grad_pool_owner: list[Unit | None] = [None, None]
        self.pool_owner: list[Unit | None] = [None] * self.pool_size
        self._next_buffer = 0
        self.cuda = dev.type == "cuda"
        # on the CPU the "prefetch" gathers run in place of the side stream: same buffer rotation, no overlap
        self.prefetch = prefetch
        self.comm_stream = torch.cuda.Stream(device=dev) if (self.prefetch and self.cuda) else None
        self.free_event: list = [None] * self.pool_size      # compute finished with the buffer's last occupant
        self.stats = {"gathers": 0, "reduce_scatters": 0, "prefetch_hits": 0}
        self._direction = 1
        self._last_index = -1
        if self.root is not None:
            self.root_params = torch.empty(self.root.numel, dtype=dt, device=dev)
            self.root_grads = torch.zeros(self.root.numel, dtype=torch.float32, device=dev)
            self._bind(self.root, self.root_params)
            self.refresh_root()
            self._install_grad_hooks(self.root, lambda: self.root_grads)
        for u in self.layer_units.values():
            self._install_grad_hooks(u, None)

    # ------------------------------------------------------------------ parameters
    def _bind(self, u: Unit, buf: torch.Tensor) -> None:
        for s, p in zip(u.slots, u.params):
            p.data = buf[s.offset:s.offset + s.numel].view(s.shape)

    def _unbind(self, u: Unit) -> None:
        for p in u.params:
            p.data = torch.empty(0, dtype=self.sp.dtype, device=self.sp.device)
        u.buffer = -1

    def refresh_root(self) -> None:
        """(Re)gathers embedding / norm / head after the shards changed (optimizer step, checkpoint load)."""
        if self.root is not None:
            _all_gather(self.root_params, self.sp.unit_shard(self.root), self.sp.group, self.sp.N)

    def _take_buffer(self, u: Unit, keep: Unit | None = None) -> int:
        """A pool buffer for ``u``, taken in rotation but never the one that holds ``keep`` (the unit that is about
        to run while ``u`` is gathered ahead: when the direction of travel turns at the top of the backward pass the
        rotation alone would hand out exactly that buffer)."""
        if self.keep_all:
            self.param_pool.append(torch.empty(u.numel, dtype=self.sp.dtype, device=self.sp.device))
            self.pool_owner.append(None)
            self.free_event.append(None)
            return len(self.param_pool) - 1
        b = self._next_buffer
        if keep is not None and self.pool_owner[b] is keep:
            b = (b + 1) % self.pool_size
        self._next_buffer = (b + 1) % self.pool_size
        old = self.pool_owner[b]
        if old is not None and old is not u:
            self._unbind(old)
        return b

    def _gather(self, u: Unit, on_side_stream: bool, keep: Unit | None = None) -> None:
        b = self._take_buffer(u, keep)
        buf = self.param_pool[b][:u.numel]
        self.stats["gathers"] += 1
        if on_side_stream:
            # the side stream may only overwrite the buffer after the compute stream finished with its last occupant
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                _all_gather(buf, self.sp.unit_shard(u), self.sp.group, self.sp.N)
                u.ready = torch.cuda.Event()
                u.ready.record(self.comm_stream)
        else:
            _all_gather(buf, self.sp.unit_shard(u), self.sp.group, self.sp.N)
            u.ready = None
        u.buffer = b
        self.pool_owner[b] = u
        self._bind(u, buf)

    def _ensure(self, u: Unit) -> None:
        if u.buffer >= 0 and self.pool_owner[u.buffer] is u:
            if u.ready is not None:
                torch.cuda.current_stream().wait_event(u.ready)
                u.ready = None
                self.stats["prefetch_hits"] += 1
            return
        self._gather(u, on_side_stream=False)

    def run(self, layer, idx: int, h, seq):
        u = self.layer_units.get(idx)
        if u is None:
            return layer(h, seq)
        # direction of travel: forward passes walk up, recomputation inside the backward pass walks down
        if idx > self._last_index:
            self._direction = 1
        elif idx < self._last_index:
            self._direction = -1
        self._last_index = idx
        self._ensure(u)
        nxt = self.layer_units.get(idx + self._direction)
        if self.prefetch and not self.keep_all and nxt is not None and not (
                nxt.buffer >= 0 and self.pool_owner[nxt.buffer] is nxt):
            self._gather(nxt, on_side_stream=self.comm_stream is not None, keep=u)
        if u.params and u.params[0].numel() == 0:
            raise RuntimeError(f"parameter-sharding runtime: layer {idx} is about to run without its parameters")
        return layer(h, seq)

    def before_forward(self) -> None:
        self._last_index, self._direction = -1, 1
        # without activation recomputation the parameters a forward pass saved must outlive it
        self.keep_all = self.model.ac_every is None and self.model.training and torch.is_grad_enabled()
        if self.keep_all:
            for u in self.layer_units.values():       # drop last step's whole units: their values are stale
                if u.buffer >= self.pool_size:
                    self._unbind(u)
            del self.param_pool[self.pool_size:], self.pool_owner[self.pool_size:], self.free_event[self.pool_size:]

    # ------------------------------------------------------------------ gradients
    def _install_grad_hooks(self, u: Unit, fixed_buffer) -> None:
        for s, p in zip(u.slots, u.params):
            def hook(param, u=u, s=s, fixed_buffer=fixed_buffer):
                g = param.grad
                param.grad = None
                buf = fixed_buffer() if fixed_buffer is not None else self._grad_buffer(u)
                if g is not None:
                    buf[s.offset:s.offset + s.numel].view(s.shape).add_(g)
                if fixed_buffer is None:
                    u.pending -= 1
                    if u.pending == 0:
                        self._reduce_unit(u)
            p.register_post_accumulate_grad_hook(hook)

    def _grad_buffer(self, u: Unit) -> torch.Tensor:
        if u.grad_buffer < 0:
            for i, owner in enumerate(self.grad_pool_owner):
                if owner is None:
                    break
            else:                                   # both in use (a unit whose parameters did not all get gradients)
                i = 0
                self._reduce_unit(self.grad_pool_owner[0])
            self.grad_pool_owner[i] = u
            u.grad_buffer = i
            u.pending = len(u.params)
        return self.grad_pool[u.grad_buffer]

    def _keep(self, u: Unit, mine: torch.Tensor) -> None:
        """This rank's reduced slice of a unit joins the persistent accumulator on the device, or leaves for the
        host accumulator when a sink is installed (``sp.grad_sink(offset, slice)``, the CPU-optimizer path)."""
        sink = getattr(self.sp, "grad_sink", None)
        if sink is not None:
            sink(u.shard_offset, mine)
        else:
            self.sp.unit_shard(u, self.sp.grad_shard).add_(mine)

    def _reduce_unit(self, u: Unit) -> None:
        """Reduce-scatter of the unit's gradient buffer; this rank's slice joins the persistent accumulator."""
        if u.grad_buffer < 0:
            return
        full = self.grad_pool[u.grad_buffer][:u.numel]
        n = u.numel // self.sp.N
        mine = torch.empty(n, dtype=torch.float32, device=self.sp.device)
        _reduce_scatter(mine, full, self.sp.group, self.sp.N)
        self._keep(u, mine)
        full.zero_()
        self.grad_pool_owner[u.grad_buffer] = None
        u.grad_buffer, u.pending = -1, 0
        self.stats["reduce_scatters"] += 1

    def finish_backward(self) -> None:
        """End of the step's last backward pass: flush units that are still holding gradients and the root."""
        for u in self.layer_units.values():
            if u.grad_buffer >= 0:
                self._reduce_unit(u)
        if self.root is not None:
            n = self.root.numel // self.sp.N
            mine = torch.empty(n, dtype=torch.float32, device=self.sp.device)
            _reduce_scatter(mine, self.root_grads, self.sp.group, self.sp.N)
            self._keep(self.root, mine)
            self.root_grads.zero_()

    def after_optimizer_step(self) -> None:
        """The shards changed: whole units still bound to a pool buffer are stale."""
        for u in self.layer_units.values():
            if u.buffer >= 0:
                self.pool_owner[u.buffer] = None
                self._unbind(u)
        self.refresh_root()

    # ------------------------------------------------------------------ whole-model access
    @contextlib.contextmanager
    def full_parameters(self, writeback: bool = False):
        """All parameters whole at once (checkpoints, weight export). With ``writeback`` the values present at
        exit are re-sharded into the persistent storage (checkpoint load)."""
        held = []
        with torch.no_grad():
            for u in self.layer_units.values():
                if u.buffer >= 0:
                    self.pool_owner[u.buffer] = None
                full = torch.empty(u.numel, dtype=self.sp.dtype, device=self.sp.device)
                _all_gather(full, self.sp.unit_shard(u), self.sp.group, self.sp.N)
                self._bind(u, full)
                held.append((u, full))
            try:
                yield
            finally:
                units = held + ([(self.root, self.root_params)] if self.root is not None else [])
                for u, full in units:
                    if writeback:
                        n = u.numel // self.sp.N
                        self.sp.unit_shard(u).copy_(full[self.sp.rank * n:(self.sp.rank + 1) * n])
                for u, _ in held:
                    self._unbind(u)


def install_fsdp(model, group, *, pool: int = 2, prefetch: bool = True) -> tuple[ShardedParameters, FSDPRuntime]:
    """Shards every trainable parameter of ``model`` that is not expert-parallel (those are already spread
    over the ep group) and installs the gather / reduce-scatter hooks."""
    layer_named: dict[int, list] = {}
    root_named: list = []
    import re

    pat = re.compile(r"^model\.layers\.(\d+)\.")
    for name, p in model.named_parameters():
        if getattr(p, "_is_expert_shard", False) or not p.requires_grad:
            continue
        m = pat.match(name)
        if m:
            layer_named.setdefault(int(m.group(1)), []).append((name, p))
        else:
            root_named.append((name, p))
    units = [(-1, root_named)] + [(i, layer_named[i]) for i in sorted(layer_named)]
    sp = ShardedParameters(units, group)
    rt = FSDPRuntime(model, sp, pool=pool, prefetch=prefetch)
    model.layer_hooks = rt
    return sp, rt
