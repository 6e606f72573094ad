"""Multi-GPU check of the context-parallel attention whose K / V exchange runs inside the
flash-attention kernel, against the all-gather (NCCL) path: outputs and gradients of q, k, v on
a packed two-document stream, then timings of forward + backward at a long sequence.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m tests.distributed.cp_attention
"""

from __future__ import annotations

import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.parallel.cp import ContextParallel


def _run(cp, q, k, v, seq, dout):
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    out = cp.attention(q, k, v, seq)
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    base = ContextParallel(group, world, rank, style="ring", layout="contiguous")      # the layout of the fused path
    fused = ContextParallel(group, world, rank, style="ring", fused_kv_gather=True)

    def setup(Tl, Hq, Hkv, lens):
        torch.manual_seed(100 + rank)
        T = Tl * world
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        assert int(cu[-1]) == T
        seq = SimpleNamespace(full_len=T, full_cu_seqlens=cu.to(dev))
        mk = lambda h: torch.randn(Tl, h, 128, device=dev).bfloat16()
        return mk(Hq), mk(Hkv), mk(Hkv), seq, mk(Hq)

    Tl = 1152
    T = Tl * world
    q, k, v, seq, dout = setup(Tl, 8, 2, [T // 2 - 77, T - (T // 2 - 77)])
    ref = _run(base, q, k, v, seq, dout)
    got = _run(fused, q, k, v, seq, dout)
    got2 = _run(fused, q, k, v, seq, dout)                 # the buffers and epochs are reused
    torch.cuda.synchronize()
    rt.check_status()
    errs = [float((a.float() - b.float()).abs().max()) for a, b in zip(ref, got)]
    errs += [float((a.float() - b.float()).abs().max()) for a, b in zip(ref, got2)]
    t = torch.tensor([max(errs)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t) < 2e-2
    if rank == 0:
        print(("CP_FUSED_OK" if ok else "CP_FUSED_FAIL"), "max deviation (out, dq, dk, dv, twice)", errs, flush=True)
    if ok and os.environ.get("CP_SELFTEST_TIMING", "1") == "1":
        Tl = 16384
        q, k, v, seq, dout = setup(Tl, 32, 4, [Tl * world])
        for name, cp in (("NCCL all-gather of K / V, then attention", base), ("K / V gathered inside the attention kernel", fused)):
            for _ in range(2):
                _run(cp, q, k, v, seq, dout)
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                _run(cp, q, k, v, seq, dout)
            e.record()
            torch.cuda.synchronize()
            rt.check_status()
            ms = torch.tensor([s.elapsed_time(e) / 5], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(f"CP_TIMING {name}: {float(ms):.3f} ms forward + backward ({Tl} local tokens x {world} ranks, "
                      f"32 / 4 heads, max over ranks)", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
