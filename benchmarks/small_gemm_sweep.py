"""Decode-sized dense bf16 GEMMs: the tcgen05 kernel's tile widths and split-K counts against the library GEMM.

    python benchmarks/small_gemm_sweep.py

For every shape: microseconds (median of CUDA-event timings with the L2 flushed between calls) of cuBLAS, of
the kernel's own choice ("auto") and of every forced (tile width, splits) pair. Forced pairs that the host
rejects (an empty split, too little workspace) fall back to one split and repeat that time.
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from prime_rl_b200.ops import _runtime as rt  # noqa: E402
from prime_rl_b200.ops import matmul as G  # noqa: E402

SHAPES = [(256, 5120, 2048), (256, 2048, 4096), (256, 128, 2048), (64, 5120, 2048), (512, 5120, 2048),
          (256, 2560, 2048), (256, 2048, 2048), (256, 151936, 2048)]


def main() -> None:
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    for M, N, K in SHAPES:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        row = [f"{M}x{N}x{K}: cublas {timed(lambda: torch.matmul(a, b.t(), out=out)):.1f} us",
               f"auto {timed(lambda: G.gemm(a, b, out=out)):.1f}"]
        if N < 100000:
            for bn in (256, 128, 64):
                for s in (1, 2, 3, 4, 6, 8):
                    row.append(f"bn{bn}s{s} {timed(lambda: G.gemm(a, b, out=out, force_bn=bn, splitk=s), n=10):.1f}")
        print("  ".join(row), flush=True)
    rt.check_status()


if __name__ == "__main__":
    main()
