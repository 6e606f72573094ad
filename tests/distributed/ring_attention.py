"""Multi-GPU check of the ring form of context-parallel attention (K / V blocks step by step, partial results merged
through the log-sum-exp, dK / dV partials returned to the owners) against the all-gather path on the same zig-zag
token layout: outputs and gradients of q, k, v on a packed stream of several documents, with the blocks relayed by
NCCL point-to-point calls and pulled from symmetric memory; then timings of forward + backward at a long sequence.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m tests.distributed.ring_attention
"""

from __future__ import annotations

import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.parallel.cp import ContextParallel


def _run(cp, q, k, v, seq, dout, window=None):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out = cp.attention(q, k, v, seq, window=window)
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    base = ContextParallel(group, world, rank, style="ring")
    relay = ContextParallel(group, world, rank, style="ring", kv_exchange="ring")
    symm = ContextParallel(group, world, rank, style="ring", kv_exchange="ring_p2p")

    def setup(Tl, Hq, Hkv, lens):
        torch.manual_seed(100 + rank)
        T = Tl * world
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        assert int(cu[-1]) == T
        seq = SimpleNamespace(full_len=T, full_cu_seqlens=cu.to(dev))
        mk = lambda h: torch.randn(Tl, h, 128, device=dev).bfloat16()
        return mk(Hq), mk(Hkv), mk(Hkv), seq, mk(Hq)

    Tl = 1152                                   # chunks of 576 rows: their edges fall inside the kernels' 128-row tiles
    T = Tl * world
    worst = 0.0
    for lens, window in (([T // 2 - 77, 300, T - (T // 2 - 77) - 300], None), ([T], 700)):
        q, k, v, seq, dout = setup(Tl, 8, 2, lens)
        ref = _run(base, q, k, v, seq, dout, window)
        for cp in (relay, symm, symm):          # the symmetric buffers and their epochs are reused
            got = _run(cp, q, k, v, seq, dout, window)
            torch.cuda.synchronize()
            rt.check_status()
            for a, b in zip(ref, got):
                worst = max(worst, float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)))
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 2e-2
    if rank == 0:
        print(("RING_ATTN_OK" if ok else "RING_ATTN_FAIL"), f"largest relative deviation {float(t):.4f}", flush=True)
    if ok and os.environ.get("CP_SELFTEST_TIMING", "1") == "1":
        Tl = 65536 // world
        q, k, v, seq, dout = setup(Tl, 32, 8, [Tl * world])
        for name, cp in (("all-gather of K / V (NCCL), one call per query slice", base),
                         ("ring, blocks relayed by NCCL point-to-point", relay),
                         ("ring, blocks pulled from symmetric memory on a side stream", symm)):
            for _ in range(2):
                _run(cp, q, k, v, seq, dout)
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(3):
                _run(cp, q, k, v, seq, dout)
            e.record()
            torch.cuda.synchronize()
            rt.check_status()
            mine = s.elapsed_time(e) / 3
            ms = torch.tensor([mine], device=dev)
            lo = torch.tensor([mine], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            if rank == 0:
                print(f"RING_TIMING {name}: {float(ms):.3f} ms forward + backward (max over ranks; fastest rank "
                      f"{float(lo):.3f} ms; 65536 tokens over {world} ranks, 32 / 8 heads)", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
