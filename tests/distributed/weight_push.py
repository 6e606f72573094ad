"""Two-GPU self test and timing of the peer-memory weight push (one process per GPU; rank 1
plays the engine, rank 0 the trainer):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29535 -m tests.distributed.weight_push

Checks that bf16 pushes are bit exact and that fp8 pushes match a PyTorch block quantiser, then
times a push of a Qwen3-30B-A3B-sized set of expert weights against an NCCL broadcast.
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist

from prime_rl_b200.ops import _runtime as rt
from prime_rl_b200.transports.weights.p2p import P2PWeightPort, _Mapped, manifest_path, push_state


class _Toy(torch.nn.Module):
    def __init__(self, dev, sizes):
        super().__init__()
        for i, shp in enumerate(sizes):
            self.register_parameter(f"w{i}", torch.nn.Parameter(torch.randn(*shp, device=dev).bfloat16()))


def _quant_ref(w: torch.Tensor):
    N, K = w.shape
    wf = w.float()
    pn, pk = (N + 127) // 128 * 128, (K + 127) // 128 * 128
    pad = torch.zeros(pn, pk, device=w.device)
    pad[:N, :K] = wf
    blocks = pad.view(pn // 128, 128, pk // 128, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
    q = (blocks / scale[:, None, :, None]).view(pn, pk)[:N, :K].to(torch.float8_e4m3fn)
    return q, scale


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    assert world == 2
    run_dir = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(run_dir, src=0)
    run_dir = Path(run_dir[0])
    torch.manual_seed(rank)
    ok = True
    for quant in (None, "fp8"):
        sizes = [(300, 520), (64,), (3, 256, 130)]
        model = _Toy(dev, sizes)
        if rank == 1:
            port = P2PWeightPort(model, run_dir, replica=0, quantize=quant)
        dist.barrier()
        if rank == 0:
            import json

            manifest = json.loads(manifest_path(run_dir, 0).read_text())
            mapped = _Mapped()
            push_state(dict(model.named_parameters()), manifest, mapped)
            torch.cuda.synchronize()
        dist.barrier()
        # compare: rank 0 sends its values through NCCL for the check
        for name, p in model.named_parameters():
            ref = p.data.clone()
            dist.broadcast(ref, src=0)
            if rank == 1:
                if quant == "fp8" and name in port.fp8:
                    q, s = port.fp8[name]
                    qr, sr = _quant_ref(ref.reshape(q.shape))
                    same_scale = torch.allclose(s, sr, rtol=1e-6, atol=0)
                    dq = (q.view(torch.float8_e4m3fn).float() - qr.float()).abs().max().item()
                    ok &= same_scale and dq <= 32.0      # at most one e4m3 step at the top binade
                    port.dequantize_into_model()
                    rel = ((p.data.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
                    ok &= rel < 0.07
                else:
                    ok &= bool(torch.equal(p.data, ref))
        if rank == 0:
            mapped.close()
        dist.barrier()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    ok = bool(t.item() > 0)
    if rank == 0:
        print("P2P_WEIGHTS_OK" if ok else "P2P_WEIGHTS_FAIL", flush=True)
    if ok and os.environ.get("P2P_SELFTEST_TIMING", "1") == "1":
        import json

        sizes = [(128, 1536, 2048), (128, 2048, 768)] * 4          # four layers of expert weights, 4.8 GB
        model = _Toy(dev, sizes)
        for quant in (None, "fp8"):
            if rank == 1:
                port = P2PWeightPort(model, run_dir, replica=0, quantize=quant)
            dist.barrier()
            if rank == 0:
                manifest = json.loads(manifest_path(run_dir, 0).read_text())
                mapped = _Mapped()
                tensors = dict(model.named_parameters())
                for _ in range(2):
                    push_state(tensors, manifest, mapped)
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(5):
                    nbytes = push_state(tensors, manifest, mapped)
                e.record()
                torch.cuda.synchronize()
                ms = s.elapsed_time(e) / 5
                src_bytes = sum(p.numel() * 2 for p in model.parameters())
                print(f"P2P_WEIGHTS_TIMING push {'bf16' if quant is None else 'bf16 -> fp8 (128x128 scales)'}: "
                      f"{ms:.2f} ms for {src_bytes / 2**30:.2f} GiB of bf16 parameters "
                      f"({nbytes / ms / 1e6:.0f} GB/s over NVLink, {src_bytes / ms / 1e6:.0f} GB/s of source)", flush=True)
                mapped.close()
            dist.barrier()
        # baseline: NCCL broadcast of the same tensors
        for _ in range(2):
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
        e.record()
        torch.cuda.synchronize()
        ms = torch.tensor([s.elapsed_time(e) / 5], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if rank == 0:
            src_bytes = sum(p.numel() * 2 for p in model.parameters())
            print(f"P2P_WEIGHTS_TIMING NCCL broadcast: {float(ms):.2f} ms ({src_bytes / float(ms) / 1e6:.0f} GB/s)", flush=True)
    rt.check_status()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
