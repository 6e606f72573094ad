"""Equal-split all-to-all over peer memory against NCCL ``all_to_all_single`` (one process per GPU):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m tests.distributed.p2p_a2a
"""

from __future__ import annotations

import sys

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.parallel.p2p_a2a import P2PAllToAll


def _selftest() -> int:
    """python -m torch.distributed.run --nproc-per-node N -m tests.distributed.p2p_a2a"""
    import os

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    torch.manual_seed(rank)
    ok = True
    op = P2PAllToAll(group, 8192 * 8 * 128 * 2, dev)
    for it in range(5):                       # more than two rounds: both buffers get reused
        x = torch.randn(world, 300 + it, 4, 128, device=dev).bfloat16()
        got = op(x)
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x, group=group)
        ok &= bool(torch.equal(got, ref))
    torch.cuda.synchronize()
    rt.check_status()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    ok = bool(t.item() > 0)
    if rank == 0:
        print("P2P_A2A_OK" if ok else "P2P_A2A_FAIL", flush=True)
    if ok and os.environ.get("P2P_SELFTEST_TIMING", "1") == "1":
        x = torch.randn(world, 8192 // world, 32 // world * 1, 128, device=dev).bfloat16()   # Ulysses q block
        x = torch.randn(world, 8192, 8, 128, device=dev).bfloat16()
        ref = torch.empty_like(x)
        for name, fn in (("NCCL all_to_all_single", lambda: dist.all_to_all_single(ref, x, group=group)),
                         ("peer-memory all-to-all", lambda: op(x))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(10):
                fn()
            e.record()
            torch.cuda.synchronize()
            ms = torch.tensor([s.elapsed_time(e) / 10], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                sent = x.numel() * 2 * (world - 1) / world
                print(f"P2P_A2A_TIMING {name}: {float(ms):.3f} ms ({sent / float(ms) / 1e6:.0f} GB/s sent per rank, "
                      f"{x.numel() * 2 / 2**20:.0f} MiB per rank, {world} ranks)", flush=True)
    op.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    import sys

    sys.exit(_selftest())
