"""Micro-benchmarks of the native kernels against the measured roofline of the device.

    python -m prime_rl_b200.ops.kernel_bench                      # all ops, default sizes
    python -m prime_rl_b200.ops.kernel_bench --op flash_fwd --tokens 4096 --iters 1 --warmup 1

Every number is the median of CUDA-event timings on the launching stream after warm-up, with
a 256 MB buffer written between iterations so that nothing is served from L2. Fractions are
relative to the peaks in ``MEASURED_PEAKS.json`` at the repository root when that file exists
(a plain copy for bandwidth, a cuBLAS bf16 GEMM for FLOP/s), else to 6.65 TB/s / 1.59 PFLOP/s.
The ``--iters 1 --warmup 1`` form is the small, short case meant to be run under a profiler.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import _runtime as rt


def _peaks():
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


class Timer:
    def __init__(self, iters, warmup, device):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def __call__(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        rt.check_status()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        rt.check_status()
        return sorted(ts)[len(ts) // 2]


def _report(name, ms, *, flops=None, bytes_=None, extra=""):
    hbm, tf, tag = _peaks()
    parts = [f"{name:44s} {ms:9.3f} ms"]
    if flops is not None:
        t = flops / ms / 1e9
        parts.append(f"{t:8.0f} TFLOP/s ({t / tf:.2f} {tag})")
    if bytes_ is not None:
        g = bytes_ / ms / 1e6
        parts.append(f"{g:8.0f} GB/s ({g / hbm:.2f} {tag})")
    print("  ".join(parts) + (f"  {extra}" if extra else ""), flush=True)


def bench_gemm(timer, args, dev):
    from .matmul import gemm

    shapes = [(8192, 8192, 8192), (16384, 4096, 2048), (16384, 5120, 2048), (16384, 2048, 4096)]
    if args.tokens:
        shapes = [(args.tokens, 4096, 2048)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        _report(f"gemm {M}x{N}x{K} (K-major B)", timer(lambda: gemm(a, b, out=out)), flops=2 * M * N * K)
        if not args.tokens:
            _report(f"  cuBLAS (torch.matmul) {M}x{N}x{K}", timer(lambda: torch.matmul(a, b.t(), out=out)),
                    flops=2 * M * N * K)


def bench_grouped(timer, args, dev):
    from .matmul import gemm

    T = args.tokens or 16384
    E, topk, H, I = 128, 8, 2048, 768
    rows = T * topk
    per = rows // E
    padded = (per + 127) // 128 * 128
    P = padded * E
    be = torch.arange(E, dtype=torch.int32, device=dev).repeat_interleave(padded // 128)
    x = torch.randn(P, H, device=dev).bfloat16()
    w1 = torch.randn(E, 2 * I, H, device=dev).bfloat16()
    w2 = torch.randn(E, H, I, device=dev).bfloat16()
    h = torch.randn(P, I, device=dev).bfloat16()
    t = torch.randn(P, 32, device=dev).bfloat16()
    b2 = torch.randn(E, 2 * I, 32, device=dev).bfloat16()
    _report(f"grouped gate_up {P}x{2 * I}x{H} E={E}", timer(lambda: gemm(x, w1, block_expert=be)), flops=2 * P * 2 * I * H)
    _report("  + fused rank-32 LoRA segment", timer(lambda: gemm(x, w1, block_expert=be, ext=(t, b2))),
            flops=2 * P * 2 * I * (H + 32))
    _report(f"grouped down {P}x{H}x{I} E={E}", timer(lambda: gemm(h, w2, block_expert=be)), flops=2 * P * H * I)
    dy = torch.randn(P, 2 * I, device=dev).bfloat16()
    _report("grouped input gradient of gate_up (MN-major B)", timer(lambda: gemm(dy, w1, b_mn=True, block_expert=be)),
            flops=2 * P * 2 * I * H)
    # weight gradients accumulated into the fp32 buffer (beta = 1): TMA reduce-adds from the epilogue
    from .lora import kgrouped_gemm

    offs = (torch.arange(E + 1, device=dev, dtype=torch.int32) * padded).contiguous()
    acc1 = torch.zeros(E, 2 * I, H, device=dev)
    acc2 = torch.zeros(E, H, I, device=dev)
    dh = torch.randn(P, H, device=dev).bfloat16()
    _report(f"k-grouped wgrad gate_up into fp32 ({per} rows / expert)",
            timer(lambda: kgrouped_gemm(dy, x, offs, E, out=acc1, beta=1.0)), flops=2 * P * 2 * I * H,
            bytes_=acc1.numel() * 4 + (dy.numel() + x.numel()) * 2)
    _report("k-grouped wgrad down into fp32", timer(lambda: kgrouped_gemm(dh, h, offs, E, out=acc2, beta=1.0)),
            flops=2 * P * H * I, bytes_=acc2.numel() * 4 + (dh.numel() + h.numel()) * 2)


def bench_fp8(timer, args, dev):
    from ..models.fp8 import quantize_to_fp8_blockwise
    from . import fp8

    M, N, K = args.tokens or 16384, 4096, 2048
    x = torch.randn(M, K, device=dev).bfloat16()
    w = torch.randn(N, K, device=dev).bfloat16()
    wq, ws = quantize_to_fp8_blockwise(w)
    wq = wq.view(torch.uint8)
    xq, xs = fp8.quantize_act(x)
    _report(f"fp8 block-scaled gemm {M}x{N}x{K}", timer(lambda: fp8.fp8_gemm(xq, xs, wq, ws)), flops=2 * M * N * K)
    _report(f"activation quantiser {M}x{K} (bf16 -> e4m3 + 1x128 scales)", timer(lambda: fp8.quantize_act(x)),
            bytes_=M * K * 3)
    # training: forward + input gradient of one projection, bf16 products against the fp8 path (quantisers included;
    # the fp8 copies of the weight and of its transpose are made once per optimizer step and are not timed)
    from .matmul import linear

    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_(False)
    dy = torch.randn(M, N, device=dev).bfloat16()

    def step(fn):
        y = fn(xg, wg)
        torch.autograd.grad(y, xg, dy)

    fp8.bump_weight_epoch()
    fp8.weight_fp8(wg, False), fp8.weight_fp8(wg, True)
    _report(f"linear fwd + dgrad {M}x{N}x{K}, bf16", timer(lambda: step(linear)), flops=4 * M * N * K)
    _report(f"linear fwd + dgrad {M}x{N}x{K}, fp8 (with activation / gradient quantisers)",
            timer(lambda: step(fp8.fp8_linear)), flops=4 * M * N * K)
    # decode-shaped grouped experts: 256 tokens x top-8 over 128 experts (weight-bandwidth bound)
    E, H, I = 128, 2048, 768
    P = E * 128
    be = torch.arange(E, dtype=torch.int32, device=dev)
    xp = torch.randn(P, H, device=dev).bfloat16()
    w1 = torch.randn(E, 2 * I, H, device=dev).bfloat16()
    w1q, w1s = quantize_to_fp8_blockwise(w1)
    w1q = w1q.view(torch.uint8)
    xpq, xps = fp8.quantize_act(xp)
    from .matmul import gemm

    _report("decode grouped gate_up, bf16 weights (805 MB)", timer(lambda: gemm(xp, w1, block_expert=be)),
            bytes_=w1.numel() * 2)
    _report("decode grouped gate_up, fp8 weights (403 MB)",
            timer(lambda: fp8.fp8_gemm(xpq, xps, w1q, w1s, block_expert=be)), bytes_=w1.numel())


def bench_lm_head(timer, args, dev):
    from .lm_head import fused_logprob_entropy

    T, V, H = args.tokens or 16384, 151936, 2048
    h = torch.randn(T, H, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device=dev) * 0.02).bfloat16()
    labels = torch.randint(0, V, (T,), device=dev)
    _report(f"lm head fwd (logprob+entropy) {T}x{V}x{H}",
            timer(lambda: fused_logprob_entropy(h.detach(), w, labels, None)), flops=2 * T * V * H)

    def fb():
        lp, _ = fused_logprob_entropy(h, w, labels, None)
        lp.sum().backward()

    _report("lm head fwd + bwd (dlogits, dh)", timer(fb), flops=6 * T * V * H)


def _attn_inputs(args, dev):
    T = args.tokens or 16384
    Hq, Hkv, D = 32, 4, 128
    q = torch.randn(T, Hq, D, device=dev).bfloat16()
    k = torch.randn(T, Hkv, D, device=dev).bfloat16()
    v = torch.randn(T, Hkv, D, device=dev).bfloat16()
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    return T, Hq, D, q, k, v, cu


def bench_flash_fwd(timer, args, dev):
    from . import flash_native

    T, Hq, D, q, k, v, cu = _attn_inputs(args, dev)
    fl = 4 * T * T / 2 * Hq * D
    _report(f"flash fwd causal T={T} Hq={Hq} Hkv=4 D=128", timer(lambda: flash_native.flash_fwd(q, k, v, cu)), flops=fl)


def bench_flash_bwd(timer, args, dev):
    from . import flash_native

    T, Hq, D, q, k, v, cu = _attn_inputs(args, dev)
    out, lse = flash_native.flash_fwd(q, k, v, cu)
    do = torch.randn_like(out)
    fl = 10 * T * T / 2 * Hq * D
    _report(f"flash bwd causal T={T} (dK/dV kernel + dQ kernel)",
            timer(lambda: flash_native.flash_bwd(do, q, k, v, out, lse, cu)), flops=fl,
            extra="(FLOPs counted as 5 products per block; 7 are executed)")


def bench_paged(timer, args, dev):
    from .paged import paged_decode_raw

    B, ctx, Hq, Hkv, D, page = 64, args.tokens or 4096, 32, 4, 128, 16
    blocks = (ctx + page - 1) // page
    pool = B * blocks
    kpool = torch.randn(pool, page, Hkv, D, device=dev).bfloat16()
    vpool = torch.randn(pool, page, Hkv, D, device=dev).bfloat16()
    tables = torch.arange(pool, dtype=torch.int32, device=dev).view(B, blocks)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, Hq, D, device=dev).bfloat16()
    by = 2 * B * ctx * Hkv * D * 2
    _report(f"paged decode B={B} ctx={ctx} GQA 32/4", timer(lambda: paged_decode_raw(q, kpool, vpool, tables, lens)), bytes_=by)


def bench_norm(timer, args, dev):
    from .norm import rms_norm

    T, H = args.tokens or 16384, 2048
    x = torch.randn(T, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    _report(f"rmsnorm fwd {T}x{H}", timer(lambda: rms_norm(x, w, 1e-6)), bytes_=2 * T * H * 2)


def bench_sparse_mla(timer, args, dev):
    from . import _runtime as rt

    T, H, topk = args.tokens or 4096, 128, 2048
    S = T
    q = (torch.randn(T, H, 576, device=dev) * 0.3).bfloat16()
    kv = (torch.randn(S, 576, device=dev) * 0.3).bfloat16()
    # causal-style selection: query t picks from [0, t]; early queries have empty slots
    idx = (torch.rand(T, topk, device=dev) * (torch.arange(T, device=dev)[:, None] + 1)).to(torch.int32)
    idx[:, :] = torch.where(torch.arange(topk, device=dev)[None, :] <= torch.arange(T, device=dev)[:, None], idx,
                            torch.full_like(idx, S))
    out = torch.empty(T, H, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(T, H, dtype=torch.float32, device=dev)
    st = rt.status_tensor(dev)

    def run():
        rt.check(rt.lib().prb_sparse_mla_fwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                             T, H, S, topk, 576 ** -0.5, st.data_ptr(), rt.stream_ptr(dev)),
                 "prb_sparse_mla_fwd")

    fl = 2.0 * T * H * topk * (576 + 512)
    _report(f"sparse MLA fwd T={T} H={H} top-{topk} (576 + 512 channels)", timer(run), flops=fl,
            extra="(algorithmic FLOPs; the two output halves each repeat Q K^T)")
    rt.check_status()


def bench_mixers(timer, args, dev):
    """Memory-bound helpers of the recurrent mixers (Nemotron-H 8B shapes)."""
    from . import ssm

    T, inner, ng, ns = args.tokens or 16384, 8192, 8, 128
    C = inner + 2 * ng * ns
    x = torch.randn(T, C, device=dev).bfloat16()
    w = torch.randn(C, 4, device=dev).bfloat16()
    b = torch.randn(C, device=dev).bfloat16()
    pos = (torch.arange(T, device=dev) % 4096).to(torch.int32)
    _report(f"causal conv1d fwd {T}x{C} k=4 + silu", timer(lambda: ssm.causal_conv1d(x, w, b, pos, "silu")),
            bytes_=2 * T * C * 2)
    h = torch.randn(T, inner, device=dev).bfloat16()
    g = torch.randn(T, inner, device=dev).bfloat16()
    nw = torch.ones(inner, device=dev).bfloat16()
    _report(f"gated group rmsnorm fwd {T}x{inner} groups of {inner // ng}",
            timer(lambda: ssm.gated_rms_norm(h, g, nw, 1e-5, inner // ng, "silu", True)), bytes_=3 * T * inner * 2)


def bench_sample(timer, args, dev):
    """Decode-step sampling over fp32 logits: the one-pass Gumbel-max kernel against the PyTorch sequence it
    replaced (scale, log-softmax, exp, multinomial, gather)."""
    from ..engine.sampler import sample_untruncated

    B, V = args.tokens or 256, 151936
    logits = torch.randn(B, V, device=dev)
    temp = torch.ones(B, device=dev)

    def torch_path():
        logp = torch.log_softmax(logits / temp[:, None], dim=-1)
        tok = torch.multinomial(logp.exp(), 1).squeeze(1)
        return tok, logp.gather(1, tok[:, None])

    _report(f"sampling kernel {B}x{V} fp32", timer(lambda: sample_untruncated(logits, temp)), bytes_=B * V * 4)
    _report(f"sampling, PyTorch ops {B}x{V} fp32", timer(torch_path), bytes_=B * V * 4)


OPS = {"sample": bench_sample, "gemm": bench_gemm, "sparse_mla": bench_sparse_mla, "mixers": bench_mixers, "grouped": bench_grouped, "fp8": bench_fp8, "lm_head": bench_lm_head, "flash_fwd": bench_flash_fwd,
       "flash_bwd": bench_flash_bwd, "paged": bench_paged, "norm": bench_norm}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="all", choices=["all", *OPS])
    ap.add_argument("--tokens", type=int, default=0, help="problem size override (rows / sequence length)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    timer = Timer(args.iters, args.warmup, dev)
    for name, fn in OPS.items():
        if args.op in ("all", name):
            fn(timer, args, dev)
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
