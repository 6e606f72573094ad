"""Ring form of context-parallel attention on CPU ranks (gloo): outputs and gradients against the all-gather path,
both token layouts, several documents and a sliding window. Run by tests/test_ring_attention_cpu.py with 4 ranks."""

from __future__ import annotations

import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist

from prime_rl_b200.parallel.cp import ContextParallel


def _run(cp, q, k, v, seq, dout, window):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out = cp.attention(q, k, v, seq, window=window)
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    group = dist.group.WORLD
    worst = 0.0
    for layout in ("zigzag", "contiguous"):
        base = ContextParallel(group, world, rank, style="ring", layout=layout)
        ring = ContextParallel(group, world, rank, style="ring", layout=layout, kv_exchange="ring")
        Tl = 48
        T = Tl * world
        for lens, window in (([T // 2 - 5, 30, T - (T // 2 - 5) - 30], None), ([T], 50)):
            torch.manual_seed(7 + rank)
            cu = torch.zeros(len(lens) + 1, dtype=torch.long)
            cu[1:] = torch.tensor(lens).cumsum(0)
            seq = SimpleNamespace(full_len=T, full_cu_seqlens=cu)
            q, k, v, dout = torch.randn(Tl, 4, 16), torch.randn(Tl, 2, 16), torch.randn(Tl, 2, 16), torch.randn(Tl, 4, 16)
            ref = _run(base, q, k, v, seq, dout, window)
            got = _run(ring, q, k, v, seq, dout, window)
            for a, b in zip(got, ref):
                worst = max(worst, float((a - b).abs().max()))
    t = torch.tensor([worst])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 1e-4
    if rank == 0:
        print(("RING_CPU_OK" if ok else "RING_CPU_FAIL"), float(t), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
