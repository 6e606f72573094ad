"""Two-or-more-GPU self test and timing of the peer-memory expert-parallel dispatcher against
the all-to-all baseline. Launch with one process per GPU:

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 \
        --master-addr 127.0.0.1 --master-port 29533 -m tests.distributed.ep_dispatch

Rank 0 prints ``EP_SELFTEST_OK`` with the largest deviations, then the device-timed
forward + backward of both dispatchers (max over ranks) at a Qwen3-30B-A3B-like layer shape.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from prime_rl_b200.models.config import ModelArch, PRESETS
from prime_rl_b200.models.layers import GroupedExperts
from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.ops import moe as moe_ops
from prime_rl_b200.parallel.ep import TorchA2ADispatcher
from prime_rl_b200.parallel.ep_p2p import P2PDispatcher


def _arch(E, H, I, k) -> ModelArch:
    return ModelArch(**{**PRESETS["tiny-qwen3-moe"], "num_experts": E, "hidden_size": H, "moe_intermediate_size": I,
                        "num_experts_per_tok": k})


def _run(disp, experts, x, idx, w, counts, dout):
    x = x.detach().clone().requires_grad_()
    w = w.detach().clone().requires_grad_()
    for p in experts.parameters():
        p.grad = None
    y = disp(experts, x, idx, w, counts)
    y.backward(dout)
    return y.detach(), x.grad, w.grad, [p.grad.clone() for p in experts.parameters()]


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    torch.manual_seed(1234 + rank)

    def setup(T, E, H, I, k):
        arch = _arch(E, H, I, k)
        ex = GroupedExperts(arch, num_local_experts=E // world, dtype=torch.bfloat16, device=dev)
        with torch.no_grad():
            ex.gate_up_proj.normal_(0, 0.05)
            ex.down_proj.normal_(0, 0.05)
        x = torch.randn(T, H, device=dev).bfloat16()
        logits = torch.randn(T, E, device=dev)
        idx, w, counts = moe_ops.route_topk(logits, k)
        dout = torch.randn(T, H, device=dev).bfloat16()
        return ex, x, idx.to(torch.int32).contiguous(), w.detach(), counts, dout

    # ---- numerics on a small, ragged case (some experts get no token)
    ex, x, idx, w, counts, dout = setup(T=300 + 117 * rank, E=8 * world, H=256, I=128, k=2)
    ref = _run(TorchA2ADispatcher(group, world, 8 * world), ex, x, idx, w, counts, dout)
    p2p = P2PDispatcher(group, world, 8 * world, capacity_factor=float(world), per_block=True)
    got = _run(p2p, ex, x, idx, w, counts, dout)
    got2 = _run(p2p, ex, x, idx, w, counts, dout)          # buffers and epochs are reused
    # the same with one global wait instead of the per-block arrival counters, then per-block again: the two
    # kinds of call may alternate on one set of buffers
    glob = P2PDispatcher(group, world, 8 * world, capacity_factor=float(world), per_block=False)
    got3 = _run(glob, ex, x, idx, w, counts, dout)
    got4 = _run(p2p, ex, x, idx, w, counts, dout)
    torch.cuda.synchronize()
    rt.check_status()
    errs = []
    for a, b, c, d, e in zip(ref[:3], got[:3], got2[:3], got3[:3], got4[:3]):
        errs.append(float((a.float() - b.float()).abs().max()))
        errs.append(float((a.float() - c.float()).abs().max()))
        errs.append(float((a.float() - d.float()).abs().max()))
        errs.append(float((a.float() - e.float()).abs().max()))
    for a, b in zip(ref[3], got[3]):
        errs.append(float((a.float() - b.float()).abs().max() / (a.float().abs().max() + 1e-6)))
    t = torch.tensor([max(errs)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 6e-2
    if rank == 0:
        print(("EP_SELFTEST_OK" if ok else "EP_SELFTEST_FAIL"), "max deviation", float(t), "per item", errs, flush=True)

    # ---- fp8 payload on the forward dispatch: relative deviation of outputs and gradients
    q = P2PDispatcher(group, world, 8 * world, capacity_factor=float(world), payload="fp8")
    gotq = _run(q, ex, x, idx, w, counts, dout)
    torch.cuda.synchronize()
    rt.check_status()
    rel = [float((a.float() - b.float()).norm() / (a.float().norm() + 1e-9)) for a, b in zip(ref[:3], gotq[:3])]
    tq = torch.tensor([max(rel)], device=dev)
    dist.all_reduce(tq, op=dist.ReduceOp.MAX)
    okq = float(tq) < 5e-2
    ok = ok and okq
    if rank == 0:
        print(("EP_FP8_PAYLOAD_OK" if okq else "EP_FP8_PAYLOAD_FAIL"), "relative deviation (out, dx, dw)", rel, flush=True)

    # ---- timing at a realistic layer shape
    if ok and os.environ.get("EP_SELFTEST_TIMING", "1") == "1":
        T, E, H, I, k = 8192, 128, 2048, 768, 8
        ex, x, idx, w, counts, dout = setup(T, E, H, I, k)
        for name, disp in (("all_to_all (NCCL)", TorchA2ADispatcher(group, world, E)),
                           ("peer memory, per-block arrival", P2PDispatcher(group, world, E, capacity_factor=2.0, per_block=True)),
                           ("peer memory, one global wait",
                            P2PDispatcher(group, world, E, capacity_factor=2.0, per_block=False)),
                           ("peer memory, fp8 dispatch payload",
                            P2PDispatcher(group, world, E, capacity_factor=2.0, payload="fp8"))):
            for _ in range(3):
                _run(disp, ex, x, idx, w, counts, dout)
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                _run(disp, ex, x, idx, w, counts, dout)
            e.record()
            torch.cuda.synchronize()
            rt.check_status()
            ms = torch.tensor([s.elapsed_time(e) / 5], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(f"EP_TIMING {name}: {float(ms):.3f} ms per MoE layer forward+backward "
                      f"(T={T}/rank, E={E}, top-{k}, H={H}, {world} ranks, max over ranks)", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
