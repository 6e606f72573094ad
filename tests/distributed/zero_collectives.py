"""Multi-GPU check of the sharded optimizer with peer-memory collectives against the NCCL ones:
two full-parameter RL trainer steps on a tiny dense model with ``model.optim_collectives = "p2p"``
and ``"nccl"``, same seeds; losses, gradient norms and the updated parameters must agree. Then the
two kernels are timed on 1 GiB of fp32 gradients / 512 MiB of bf16 parameters against
``reduce_scatter_tensor`` / ``all_gather_into_tensor``.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m tests.distributed.zero_collectives
"""

from __future__ import annotations

import os
import sys
import tempfile

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt


def _trainer_run(kind: str, tmp: str):
    from prime_rl_b200.configs.trainer import TrainerConfig
    from prime_rl_b200.trainer.rl.train import RLTrainer

    cfg = TrainerConfig.model_validate({
        "model": {"name": "tiny-qwen3", "seq_len": 256, "ac": None, "optim_collectives": kind,
                  "arch": {"head_dim": 128, "num_attention_heads": 2, "num_key_value_heads": 1},
                  "debug": {"random_init": True}},
        "optim": {"lr": 1e-3, "max_norm": 1.0}, "max_steps": 2, "output_dir": os.path.join(tmp, kind),
        "data": {"fake": {"batch_size": 2 * int(os.environ["WORLD_SIZE"]), "generate_samples": True}}})
    tr = RLTrainer(cfg).setup()
    out = []
    for _ in range(2):
        m = tr.step()
        out.append((m["loss"], m["optim/grad_norm"]))
    flat = tr.optimizer.buf.flat.detach().float().clone()
    used = tr.optimizer.groups[0].p2p is not None
    return out, flat, used


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from prime_rl_b200.utils.logger import setup_logger

    setup_logger("warning")
    with tempfile.TemporaryDirectory() as tmp:
        a, fa, used_a = _trainer_run("nccl", tmp)
        b, fb, used_b = _trainer_run("p2p", tmp)
    torch.cuda.synchronize()
    rt.check_status()
    dev_l = max(abs(x[0] - y[0]) for x, y in zip(a, b))
    dev_g = max(abs(x[1] - y[1]) / max(abs(x[1]), 1e-9) for x, y in zip(a, b))
    dev_p = float((fa - fb).abs().max())
    t = torch.tensor([dev_l, dev_g, dev_p, 0.0 if (used_b and not used_a) else 1.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t[0]) < 1e-5 and float(t[1]) < 1e-4 and float(t[2]) < 1e-3 and float(t[3]) == 0.0
    if rank == 0:
        print(("P2P_ZERO_OK" if ok else "P2P_ZERO_FAIL"), "deviation of (loss, grad norm, parameters), p2p used:",
              t.tolist(), flush=True)
    if ok and os.environ.get("P2P_ZERO_TIMING", "1") == "1":
        from prime_rl_b200.parallel.p2p_zero import P2PShardCollectives

        group = dist.group.WORLD
        n = 256 * 1024 * 1024                       # 1 GiB of fp32 gradients, 512 MiB of bf16 parameters
        coll = P2PShardCollectives(group, n, torch.bfloat16, dev)
        coll.grad.normal_()
        shard = torch.empty(n // world, dtype=torch.float32, device=dev)
        flat2 = torch.empty(n, dtype=torch.bfloat16, device=dev)

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                fn()
            e.record()
            torch.cuda.synchronize()
            ms = torch.tensor([s.elapsed_time(e) / 5], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms)

        lo, ln = rank * (n // world), n // world
        rows = [("reduce-scatter 1 GiB fp32: NCCL", lambda: dist.reduce_scatter_tensor(shard, coll.grad, group=group)),
                ("reduce-scatter 1 GiB fp32: peer loads + scale", lambda: coll.reduce_scatter(shard, lo, 0.5)),
                ("all-gather 512 MiB bf16: NCCL", lambda: dist.all_gather_into_tensor(flat2, flat2[lo:lo + ln], group=group)),
                ("all-gather 512 MiB bf16: peer stores", lambda: coll.all_gather(lo, ln))]
        for name, fn in rows:
            ms = timed(fn)
            if rank == 0:
                print(f"P2P_ZERO_TIMING {name}: {ms:.3f} ms ({world} ranks, max over ranks)", flush=True)
        rt.check_status()
        coll.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
