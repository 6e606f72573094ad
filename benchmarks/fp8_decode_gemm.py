"""Times the two grouped block-scaled fp8 GEMMs of one MoE layer at decode size (a handful of rows per expert,
padding rows masked).

    python benchmarks/fp8_decode_gemm.py [--tokens 256] [--experts 128] [--topk 8] [--hidden 2048] [--inter 768]

Prints microseconds per call (CUDA events, L2 flushed between calls) and the weight bytes / time as a fraction
of the copy bandwidth given with --hbm-gbs.
"""

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from prime_rl_b200.ops import _runtime as rt  # noqa: E402
from prime_rl_b200.ops import fp8, moe  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=6650.0)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    T, E, k, H, I = args.tokens, args.experts, args.topk, args.hidden, args.inter
    logits = torch.randn(T, E, device=dev)
    idx, w, counts = moe.route_topk(logits, k)
    plan = moe.build_plan(idx.to(torch.int32).contiguous(), counts.to(torch.int32), E)
    P = plan.max_rows
    valid = plan.row_src
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def quant_w(n, kk):
        wq = torch.randint(0, 120, (E, n, kk), dtype=torch.uint8, device=dev)
        ws = torch.rand(E, (n + 127) // 128, (kk + 127) // 128, device=dev) * 0.01 + 0.001
        return wq, ws

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    for name, n, kk in (("gate_up", 2 * I, H), ("down", H, I)):
        wq, ws = quant_w(n, kk)
        x = torch.randn(P, kk, device=dev).bfloat16()
        xq, xs = fp8.quantize_act(x)
        out = torch.empty(P, n, dtype=torch.bfloat16, device=dev)
        t_tile = timed(lambda: fp8.fp8_gemm(xq, xs, wq, ws, block_expert=plan.block_expert, out=out, row_valid=valid))
        wbytes = E * n * kk
        floor = wbytes / (args.hbm_gbs * 1e3)
        print(f"{name}: {T} tokens x top-{k} over {E} experts, N={n} K={kk}: {t_tile:.1f} us; weights "
              f"{wbytes / 1e6:.0f} MB = {floor:.1f} us at {args.hbm_gbs:.0f} GB/s -> {floor / t_tile:.2f} of the "
              f"copy rate", flush=True)
    rt.check_status()


if __name__ == "__main__":
    main()
