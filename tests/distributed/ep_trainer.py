"""Two-GPU end-to-end check of expert parallelism inside the RL trainer: one optimizer step of a
small MoE model with experts sharded over 2 ranks, once with the all-to-all dispatcher and once
with the peer-memory dispatcher; losses and gradient norms must agree.

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 \
        --master-addr 127.0.0.1 --master-port 29537 -m tests.distributed.ep_trainer
"""

from __future__ import annotations

import os
import sys
import tempfile

import torch
import torch.distributed as dist


def _step(dispatch: str, out_dir: str):
    from prime_rl_b200.configs.trainer import TrainerConfig
    from prime_rl_b200.trainer.rl.train import RLTrainer

    cfg = TrainerConfig.model_validate({
        "model": {"name": "qwen3-30b-a3b", "seq_len": 1024, "ep": 2,
                  "moe": {"dispatch": {"type": dispatch}},
                  "arch": {"num_hidden_layers": 2, "num_experts": 16, "vocab_size": 8192, "hidden_size": 512,
                           "num_attention_heads": 4, "num_key_value_heads": 2, "moe_intermediate_size": 256},
                  "debug": {"random_init": True}},
        "data": {"fake": {"batch_size": 2}}, "optim": {"lr": 1e-4}, "monitors": {"file": None},
        "output_dir": out_dir})
    trainer = RLTrainer(cfg).setup()
    m = trainer.step()
    torch.cuda.synchronize()
    return float(m["loss"]), float(m["optim/grad_norm"])


def main() -> int:
    from prime_rl_b200.ops import _runtime as rt

    out = tempfile.mkdtemp()
    a = _step("torch", out)
    b = _step("p2p", out)
    rt.check_status()
    rank = dist.get_rank()
    ok = abs(a[0] - b[0]) < 1e-3 * max(1.0, abs(a[0])) and abs(a[1] - b[1]) < 2e-2 * max(1e-6, abs(a[1]))
    t = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_TRAINER_OK" if t.item() > 0 else "EP_TRAINER_FAIL", "all_to_all (loss, grad norm)", a,
              "peer memory", b, flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if t.item() > 0 else 1


if __name__ == "__main__":
    sys.exit(main())
