"""Expert parallelism: experts are sharded over the ``ep`` group (contiguous ranges); tokens
travel to the rank that owns their expert and back.

``TorchA2ADispatcher`` is the library baseline (counts exchange + variable-split
``all_to_all_single``, NCCL or gloo) — the data path of the reference's
``TorchTokenDispatcher`` (src/prime_rl/trainer/distributed/token_dispatcher.py:247-301,
collectives.py:16-17), including its host read of the split sizes. The peer-memory
dispatcher in ``parallel/ep_p2p.py`` writes rows straight into the owner's expert-sorted
buffer instead and needs no host synchronisation.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import moe as moe_ops


class _AllToAll(torch.autograd.Function):
    """Variable-split all-to-all over dim 0; backward runs the transposed exchange."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = dy.new_empty((sum(ctx.in_splits),) + tuple(dy.shape[1:]))
        dist.all_to_all_single(dx, dy.contiguous(), output_split_sizes=ctx.in_splits,
                               input_split_sizes=ctx.out_splits, group=ctx.group)
        return dx, None, None, None


def all_to_all(x, out_splits, in_splits, group):
    return _AllToAll.apply(x, out_splits, in_splits, group)


class TorchA2ADispatcher:
    def __init__(self, group, ep: int, num_experts: int):
        self.group, self.ep, self.E = group, ep, num_experts
        self.E_local = num_experts // ep

    def __call__(self, experts, x, idx, w, counts):
        """x [T, H]; idx [T, k] global expert ids; w [T, k]; counts [E]. Returns y [T, H]."""
        T, k = idx.shape
        ep, El = self.ep, self.E_local
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)               # pairs sorted by global expert
        send_rows = x[order // k]                              # differentiable gather
        # counts exchange: what every rank sends to each of my local experts
        send_counts = counts.to(torch.int64).reshape(ep, El)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        in_splits = send_counts.sum(1).tolist()                # host read (baseline behaviour)
        out_splits = recv_counts.sum(1).tolist()
        recv_rows = all_to_all(send_rows, out_splits, in_splits, self.group)
        # local expert id of every received row (grouped by source rank, sorted inside)
        R = recv_rows.shape[0]
        local_ids = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(ep), recv_counts.reshape(-1),
                                            output_size=R).to(torch.int32)
        local_counts = recv_counts.sum(0).to(torch.int32)
        plan = moe_ops.build_plan(local_ids.reshape(R, 1), local_counts, El)
        xp = moe_ops.permute(recv_rows, plan)
        yp = experts(xp, plan.block_expert, plan.expert_offset)
        ones = torch.ones(R, 1, dtype=torch.float32, device=x.device)
        back = moe_ops.combine(yp, ones, plan, R)
        ret = all_to_all(back, in_splits, out_splits, self.group)   # rows in my sorted-pair order
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=x.device)
        rows = ret[inv].reshape(T, k, -1)                           # [T, k, H] in (t, j) order
        return (rows.float() * w.float()[:, :, None]).sum(1).to(x.dtype)


def install_expert_parallel(model, dims, moe_cfg=None) -> None:
    """Keeps only this rank's expert range in every MoE layer and installs the dispatcher.
    Expert parameters are tagged so that the optimizer reduces them over the ranks that hold
    the same shard (``dp_shard_mod_ep`` x ``dp_replicate``) instead of all data-parallel ranks."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    ep = dims.ep
    ep_rank = dims.coords(rank)["ep"]
    group = dims.group("ep")
    kind = getattr(getattr(moe_cfg, "dispatch", None), "type", "torch")
    model.ep_info = None
    for moe in model.moe_layers():
        E = moe.arch.num_experts
        if E % ep:
            raise ValueError(f"num_experts {E} is not divisible by ep {ep}")
        El = E // ep
        ex = moe.experts
        for name in ("gate_up_proj", "down_proj"):
            p = getattr(ex, name)
            p.data = p.data[ep_rank * El:(ep_rank + 1) * El].clone()
            p._is_expert_shard = True
        for ad in (ex.lora_gate_up, ex.lora_down):
            if ad is not None:
                ad.lora_A.data = ad.lora_A.data[ep_rank * El:(ep_rank + 1) * El].clone()
                ad.lora_A._is_expert_shard = True
                for b in ad.lora_B:
                    b.data = b.data[ep_rank * El:(ep_rank + 1) * El].clone()
                    b._is_expert_shard = True
        if kind in ("p2p", "deepep"):
            from .ep_p2p import P2PDispatcher

            dcfg = getattr(moe_cfg, "dispatch", None)
            moe.dispatcher = P2PDispatcher(group, ep, E, capacity_factor=getattr(dcfg, "capacity_factor", None),
                                           payload=getattr(dcfg, "payload", "bf16"),
                                           per_block=bool(getattr(dcfg, "per_block_arrival", False)))
        else:
            moe.dispatcher = TorchA2ADispatcher(group, ep, E)
        moe.ep_rank, moe.ep = ep_rank, ep
        if model.ep_info is None:
            # what checkpoints and weight transports need to know about the slicing; when several ep
            # groups replicate the experts, the group of global rank 0 is the one that exports them
            model.ep_info = {"ep": ep, "ep_rank": ep_rank, "group": group, "num_experts": E, "local_experts": El,
                             "writer": rank < ep, "replicas": dims.world_size // ep,
                             "replica": rank // ep, "rank_lists": dims._rank_lists("ep")}
