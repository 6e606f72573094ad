"""Tensor parallelism for the rollout engine: one process per GPU, all ranks run the same
scheduler in lockstep over the same request stream, the decoder's weights are split.

What is split (``shard_tensor``):
  attention   heads: rank r owns q heads [r nq/R, (r+1) nq/R) and their kv heads; ``o_proj`` by columns
  dense MLP   the intermediate width: gate / up rows and ``down_proj`` columns
  experts     the intermediate width of EVERY expert (all ranks route all tokens to all experts and
              read 1/R of each expert's weights: decode is bound by that read); or, with
              ``expert_parallel`` (``enable_expert_parallel`` of the inference config), whole experts:
              rank r owns experts [r E/R, (r+1) E/R) at full width. The tokens are present on every
              rank anyway (the layer input is the output of a reduction), so there is no dispatch: every
              rank routes all tokens, runs the pairs whose expert it owns (``ops/moe.py: build_plan`` with
              ``expert_range``) and the layer's reduction sums the partial outputs
Embedding, router, norms and the LM head are replicated. Each decoder layer therefore ends in two
sums over ranks (after ``o_proj`` and after the MLP); ``TPContext.reduce`` does each of them in ONE kernel
over peer memory together with the residual add and the next RMSNorm (csrc/ep_p2p.cu,
``ar_add_rmsnorm_kernel``), with a device-side call counter so that CUDA graphs can replay it.

The reference gets tensor parallelism from the serving engine it drives (``tensor_parallel_size`` in
packages/prime-rl-configs/src/prime_rl/configs/inference.py:88-97, NCCL / custom all-reduce plus
separate add-norm kernels inside vLLM).

Control plane: rank 0 owns the HTTP server; before every step it broadcasts the requests that
arrived (and admin commands) to the other ranks over a gloo group, so every rank admits, preempts
and finishes the same requests in the same order. Rank 0 samples; the tokens are broadcast.
"""

from __future__ import annotations

import re

import torch
import torch.distributed as dist

_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def _rows(t: torch.Tensor, sections: list[int], rank: int, size: int) -> torch.Tensor:
    """Slice ``rank`` of every section along dim -2 (matrices) or -1 (vectors), sections stacked."""
    dim = t.dim() - 2 if t.dim() >= 2 else 0
    out, start = [], 0
    for n in sections:
        if n % size:
            raise ValueError(f"a section of {n} rows cannot be split over {size} ranks")
        per = n // size
        out.append(t.narrow(dim, start + rank * per, per))
        start += n
    assert start == t.shape[dim], (start, tuple(t.shape))
    return torch.cat(out, dim) if len(out) > 1 else out[0]


def _cols(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = t.shape[-1]
    if n % size:
        raise ValueError(f"{n} columns cannot be split over {size} ranks")
    return t.narrow(-1, rank * (n // size), n // size)


def expert_slice(arch, rank: int, size: int) -> tuple[int, int]:
    E = arch.num_experts
    if E % size:
        raise ValueError(f"{E} experts cannot be split over {size} ranks")
    return rank * (E // size), (rank + 1) * (E // size)


def shard_tensor(name: str, t: torch.Tensor, arch, rank: int, size: int, expert_parallel: bool = False
                 ) -> torch.Tensor:
    """The part of native-layout tensor ``name`` that TP rank ``rank`` of ``size`` keeps (a view or a
    new tensor; replicated tensors are returned as they are)."""
    if size == 1:
        return t
    if expert_parallel and ".experts." in name and t.dim() >= 1 and t.shape[0] == arch.num_experts:
        lo, hi = expert_slice(arch, rank, size)
        return t[lo:hi]                                           # weights and per-expert biases alike
    m = _LAYER.search(name)
    if m is None:
        return t
    li = int(m.group(1))
    D = arch.head_dim
    nq, nkv = arch.layer_heads(li), arch.num_key_value_heads
    single = arch.hidden_act == "relu2"                       # no up half
    if ".self_attn." in name:
        if "qkv_proj." in name:
            return _rows(t, [nq * D, nkv * D, nkv * D], rank, size)
        if name.endswith("o_proj.weight"):
            return _cols(t, rank, size)
        if name.endswith("o_proj.bias"):
            return t if rank == 0 else torch.zeros_like(t)
        if "g_proj." in name:
            return _rows(t, [t.shape[0]], rank, size)
        if name.endswith(".sinks"):
            return _rows(t, [nq], rank, size)
        return t
    if name.endswith("experts.gate_up_proj"):
        I = t.shape[-2] if single else t.shape[-2] // 2
        return _rows(t, [I] if single else [I, I], rank, size)
    if name.endswith("experts.down_proj"):
        return _cols(t, rank, size)
    if "gate_up_proj." in name:                               # dense MLP and shared experts
        I = t.shape[0] if single else t.shape[0] // 2
        return _rows(t, [I] if single else [I, I], rank, size)
    if name.endswith("down_proj.weight"):
        return _cols(t, rank, size)
    if name.endswith("down_proj.bias"):
        return t if rank == 0 else torch.zeros_like(t)
    return t


def shard_model_(model, rank: int, size: int, expert_parallel: bool = False) -> None:
    """Replaces the parameters of ``model`` by this rank's shards (in place) and leaves a
    ``model.tp_shard(name, tensor)`` hook that later weight loads go through."""
    from ..models.layers import Attention, DecoderLayer, MoE

    arch = model.arch
    if size == 1:
        return
    if arch.num_key_value_heads % size or any(arch.layer_heads(i) % size for i in range(arch.num_hidden_layers)):
        raise ValueError(f"{arch.num_key_value_heads} kv heads cannot be split over {size} ranks")
    for layer in model.model.layers:
        if not isinstance(layer, DecoderLayer) or not isinstance(layer.self_attn, Attention):
            raise NotImplementedError("engine tensor parallelism covers the attention + MLP/MoE decoder families")
    with torch.no_grad():
        for name, p in list(model.named_parameters()):
            if "lora_" in name:
                raise NotImplementedError("merge or drop LoRA adapters before sharding the engine's model")
            new = shard_tensor(name, p.data, arch, rank, size, expert_parallel)
            if new is not p.data:
                p.data = new.contiguous()
    for layer in model.model.layers:
        at = layer.self_attn
        at.nq, at.nkv = at.nq // size, at.nkv // size
        if expert_parallel and isinstance(layer.mlp, MoE):
            layer.mlp.expert_range = expert_slice(arch, rank, size)
    model.tp_shard = lambda name, t: shard_tensor(name, t, arch, rank, size, expert_parallel)
    model.tp_size, model.tp_rank, model.tp_expert_parallel = size, rank, expert_parallel


class TPContext:
    """Symmetric partial-sum buffers + flags of one TP group and the fused reduce kernel."""

    def __init__(self, group, device: torch.device, hidden: int, max_tokens: int, control_group=None):
        from ..ops import _runtime as rt
        from ..parallel.symm import SymmetricBuffer

        self.group, self.device, self.hidden = group, device, hidden
        self.control = control_group
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.max_tokens = max_tokens
        self.buf_bytes = (max_tokens * hidden * 2 + 255) // 256 * 256
        self.symm = SymmetricBuffer(group, 2 * self.buf_bytes + 256, device)
        self.buf_ptrs = [self.symm.offset_ptrs(0), self.symm.offset_ptrs(self.buf_bytes)]
        self.flag_ptrs = self.symm.offset_ptrs(2 * self.buf_bytes)
        self.bufs = [self.symm.local(torch.bfloat16, 0, max_tokens * hidden).view(max_tokens, hidden),
                     self.symm.local(torch.bfloat16, self.buf_bytes, max_tokens * hidden).view(max_tokens, hidden)]
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        self.calls = 0
        self._rt = rt

    def reduce(self, partial: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor | None, eps: float):
        """``partial`` [rows, hidden] bf16 of this rank -> (rmsnorm(sum + residual) * weight, sum + residual);
        the first is None without ``weight``."""
        rt = self._rt
        rows = partial.shape[0]
        if rows > self.max_tokens:
            raise ValueError(f"{rows} rows exceed the {self.max_tokens} the tensor-parallel buffers were sized for")
        b = self.calls & 1
        self.calls += 1
        self.bufs[b][:rows].copy_(partial)
        out_h = torch.empty(rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        out_x = torch.empty_like(out_h) if weight is not None else None
        rt.check(rt.lib().prb_ar_add_rmsnorm(self.buf_ptrs[b], self.flag_ptrs, self.state.data_ptr(),
                                             residual.data_ptr() if residual is not None else None,
                                             weight.data_ptr() if weight is not None else None, out_h.data_ptr(),
                                             out_x.data_ptr() if out_x is not None else None, rows, self.hidden,
                                             float(eps), self.rank, self.size, rt.status_tensor(self.device).data_ptr(),
                                             rt.stream_ptr(self.device)), "prb_ar_add_rmsnorm")
        return out_x, out_h

    def broadcast_sample(self, tok: torch.Tensor, lp: torch.Tensor):
        packed = torch.stack([tok.double(), lp.double()])
        dist.broadcast(packed, src=dist.get_global_rank(self.group, 0), group=self.group)
        return packed[0].long(), packed[1].float()

    def broadcast_control(self, msg):
        """Rank 0 passes ``msg`` (picklable); the others pass None and get rank 0's message."""
        box = [msg]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.control or self.group)
        return box[0]

    def close(self):
        self.symm.close()


def init_tp(max_tokens: int, hidden: int):
    """Process-group setup for a launch with one process per GPU (``torchrun`` environment): NCCL group
    for the data plane, gloo group for the control messages. Returns a ``TPContext``."""
    import datetime
    import os

    if not torch.cuda.is_available():           # CPU: gloo for both planes, PyTorch arithmetic
        if not dist.is_initialized():
            dist.init_process_group("gloo", timeout=datetime.timedelta(days=2))
        return CollectiveTPContext(dist.group.WORLD, torch.device("cpu"), hidden, max_tokens)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    control = dist.new_group(backend="gloo", timeout=datetime.timedelta(days=2))
    return TPContext(dist.group.WORLD, dev, hidden, max_tokens, control_group=control)


class CollectiveTPContext:
    """Same interface as ``TPContext`` on plain collectives and PyTorch arithmetic: what the CPU (gloo)
    tests of the sharding and of the lockstep control plane run on."""

    def __init__(self, group, device: torch.device, hidden: int, max_tokens: int, control_group=None):
        self.group, self.device, self.hidden, self.max_tokens = group, device, hidden, max_tokens
        self.control = control_group
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.calls = 0

    def reduce(self, partial, residual, weight, eps):
        from ..ops.norm import rms_norm_ref

        self.calls += 1
        total = partial.clone()
        dist.all_reduce(total, group=self.group)
        h = total if residual is None else total + residual
        return (rms_norm_ref(h, weight, eps) if weight is not None else None), h

    broadcast_sample = TPContext.broadcast_sample
    broadcast_control = TPContext.broadcast_control

    def close(self):
        pass
