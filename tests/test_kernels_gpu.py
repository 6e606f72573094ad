"""Numerics of the sm_100a kernels against fp32 PyTorch references of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from prime_rl_b200.ops import _runtime as rt  # noqa: E402
from prime_rl_b200.ops import activation, lm_head, moe, norm, optim, rope
from prime_rl_b200.ops import matmul as G  # noqa: E402

DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (tol {atol}+{rtol}*|ref|), shape {tuple(a.shape)}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 520, 264), (77, 72, 40), (4096, 2048, 1024)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    if a_mn and M % 8:
        pytest.skip("MN-major A needs a 16-byte row pitch")
    if b_mn and N % 8:
        pytest.skip("MN-major B needs a 16-byte row pitch")
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    ref = G.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    rt.check_status()
    _close(out, ref, atol=1e-2 * K ** 0.5 / 8, rtol=1e-2)
    out_bf = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    rt.check_status()
    _close(out_bf, ref, atol=0.02 * K ** 0.5, rtol=2e-2)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths_and_beta(bn):
    M, N, K = 640, 768, 320
    a, b = _rand(M, K), _rand(N, K)
    c0 = torch.randn(M, N, device=DEV)
    ref = 0.5 * (a.float() @ b.float().t()) + 2.0 * c0
    out = c0.clone()
    G.gemm(a, b, out=out, alpha=0.5, beta=2.0, force_bn=bn)
    rt.check_status()
    _close(out, ref, atol=0.05, rtol=1e-2)


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 4, 8])
@pytest.mark.parametrize("M,N,K,b_mn", [(256, 5120, 2048, False), (77, 520, 1096, False), (512, 2048, 4096, True),
                                        (32, 128, 768, False)])
def test_gemm_split_k_for_decode_sized_outputs(M, N, K, b_mn, splits):
    """Few output tiles: the reduction is dealt to several CTAs per tile whose fp32 partials the last arrival adds
    in split order. Every split count (0 = the kernel's own choice) must give the unsplit result; twice in a row,
    because the arrival counters must be back at zero after a launch."""
    a = _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    ref = G.gemm_ref(a, b, b_mn=b_mn, out_dtype=torch.float32)
    for _ in range(2):
        out = G.gemm(a, b, b_mn=b_mn, out_dtype=torch.float32, splitk=splits)
        rt.check_status()
        _close(out, ref, atol=1e-2 * K ** 0.5 / 8, rtol=1e-2)
    c0 = torch.randn(M, N, device=DEV).to(torch.bfloat16)
    out = c0.clone()
    G.gemm(a, b, b_mn=b_mn, out=out, alpha=0.5, beta=1.0, splitk=splits)
    rt.check_status()
    _close(out, 0.5 * ref + c0.float(), atol=0.02 * K ** 0.5, rtol=2e-2)
    again = c0.clone()
    G.gemm(a, b, b_mn=b_mn, out=again, alpha=0.5, beta=1.0, splitk=splits)
    assert torch.equal(out, again)                      # partials are added in a fixed order


def test_gemm_grouped_fwd_and_dgrad():
    E, N, K = 6, 384, 256
    counts = torch.tensor([130, 0, 5, 256, 127, 1], dtype=torch.int32)
    padded = (counts + 127) // 128 * 128
    P = int(padded.sum()) + 256
    block_expert = torch.full((P // 128,), -1, dtype=torch.int32)
    blk = 0
    for e in range(E):
        for _ in range(int(padded[e]) // 128):
            block_expert[blk] = e
            blk += 1
    x = _rand(P, K)
    w = _rand(E, N, K, scale=0.1)
    be = block_expert.to(DEV)
    ref = G.grouped_gemm_ref(x, w, block_expert, out_dtype=torch.float32)
    out = G.gemm(x, w, block_expert=be, out_dtype=torch.float32)
    rt.check_status()
    used = blk * 128
    _close(out[:used], ref[:used], atol=0.03, rtol=1e-2)
    dy = _rand(P, N)
    ref_dx = G.grouped_gemm_ref(dy, w, block_expert, b_mn=True, out_dtype=torch.float32)
    dx = G.gemm(dy, w, b_mn=True, block_expert=be, out_dtype=torch.float32)
    rt.check_status()
    _close(dx[:used], ref_dx[:used], atol=0.05, rtol=1e-2)


def test_linear_autograd():
    x = _rand(300, 512).requires_grad_()
    w = _rand(384, 512, scale=0.05).requires_grad_()
    y = G.linear(x, w)
    dy = _rand(300, 384)
    y.backward(dy)
    rt.check_status()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    _close(y, yr, atol=0.05, rtol=2e-2)
    _close(x.grad, xr.grad, atol=0.05, rtol=2e-2)
    _close(w.grad, wr.grad, atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("T,V,H", [(256, 1024, 256), (300, 5000, 512), (1024, 32000, 1024)])
def test_fused_lm_head(T, V, H):
    h = _rand(T, H).requires_grad_()
    w = _rand(V, H, scale=0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    inv_temp = (0.5 + torch.rand(T, device=DEV))
    lp, ent = lm_head.fused_logprob_entropy(h, w, labels, inv_temp)
    rt.check_status()
    g = torch.randn(T, device=DEV)
    (lp * g).sum().backward()
    rt.check_status()
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    lpr, entr = lm_head.logprob_entropy_ref(hr, wr, labels, inv_temp)
    (lpr * g).sum().backward()
    _close(lp, lpr, atol=2e-2, rtol=1e-2)
    _close(ent, entr, atol=2e-2, rtol=1e-2)
    # dlogits are rounded to bf16 before the two gradient GEMMs: compare in norm
    for got, want in ((h.grad, hr.grad), (w.grad, wr.grad)):
        rel = (got.float() - want).norm() / want.norm()
        assert rel < 2e-2, f"relative error {rel:.4f}"


@pytest.mark.parametrize("rows,cols", [(33, 256), (1000, 2048), (257, 4096), (64, 128), (50, 1024)])
def test_rmsnorm(rows, cols):
    x = _rand(rows, cols).requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = norm.rms_norm(x, w, 1e-6)
    dy = _rand(rows, cols)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = norm.rms_norm_ref(xr, wr, 1e-6)
    yr.backward(dy.float())
    _close(y, yr, atol=2e-2, rtol=1e-2)
    _close(x.grad, xr.grad, atol=3e-2, rtol=2e-2)
    _close(w.grad, wr.grad, atol=0.05 * rows ** 0.5, rtol=2e-2)


def test_add_rmsnorm():
    rows, cols = 300, 2048
    x, r = _rand(rows, cols).requires_grad_(), _rand(rows, cols).requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(torch.bfloat16).requires_grad_()
    y, h = norm.add_rms_norm(x, r, w, 1e-6)
    dy, dh = _rand(rows, cols), _rand(rows, cols)
    (y * dy).sum().backward(retain_graph=True)
    gx_y = x.grad.clone()
    x.grad = None
    r.grad = None
    w.grad = None
    torch.autograd.backward([y, h], [dy, dh])
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    hr = (xr + rr)
    yr = norm.rms_norm_ref(hr.to(torch.bfloat16).float(), wr, 1e-6)
    torch.autograd.backward([yr, hr], [dy.float(), dh.float()])
    _close(y, yr, atol=3e-2, rtol=2e-2)
    _close(h, hr, atol=2e-2, rtol=1e-2)
    _close(x.grad, xr.grad, atol=5e-2, rtol=2e-2)
    _close(r.grad, xr.grad, atol=5e-2, rtol=2e-2)
    assert gx_y is not None


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("with_norm", [True, False])
def test_qknorm_rope(D, with_norm):
    T, Hh = 200, 6
    x = _rand(T, Hh, D).requires_grad_()
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_() if with_norm else None
    pos = torch.randint(0, 4096, (T,), device=DEV, dtype=torch.int32)
    inv_f = rope.inv_freq(D, 1e6, device=DEV)
    y = rope.qknorm_rope(x, w, pos, inv_f, 1e-6)
    dy = _rand(T, Hh, D)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_() if with_norm else None
    yr = rope.qknorm_rope_ref(xr, wr, pos, inv_f, 1e-6)
    yr.backward(dy.float())
    _close(y, yr, atol=3e-2, rtol=2e-2)
    _close(x.grad, xr.grad, atol=5e-2, rtol=3e-2)
    if with_norm:
        _close(w.grad, wr.grad, atol=0.6, rtol=3e-2)


@pytest.mark.parametrize("act", [activation.SWIGLU, activation.SWIGLU_CLAMPED, activation.RELU2])
def test_glu(act):
    rows, I = 123, 768
    width = I if act == activation.RELU2 else 2 * I
    gu = _rand(rows, width, scale=2.0).requires_grad_()
    y = activation.glu(gu, act)
    dy = _rand(rows, I)
    y.backward(dy)
    gur = gu.detach().float().requires_grad_()
    if act == activation.RELU2:
        yr = activation.glu_ref(gur, None, act)
    else:
        yr = activation.glu_ref(gur[:, :I], gur[:, I:], act)
    yr.backward(dy.float())
    _close(y, yr, atol=3e-2, rtol=2e-2)
    _close(gu.grad, gur.grad, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_adamw_flat(grad_dtype):
    n = 100003
    p = torch.randn(n, device=DEV)
    m = torch.randn(n, device=DEV) * 0.01
    v = torch.rand(n, device=DEV) * 0.01
    g = torch.randn(n, device=DEV).to(grad_dtype)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lowp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    step, lr, b1, b2, eps, wd = 3, 1e-3, 0.9, 0.95, 1e-8, 0.1
    ss = torch.zeros(1, device=DEV)
    optim.sumsq(g, ss)
    coef, gnorm = optim.clip_coef(ss, 1.0)
    hyper = torch.tensor([lr, 1 - b1 ** step, (1 - b2 ** step) ** 0.5], device=DEV)
    optim.adamw_flat(p, m, v, g, lowp, hyper, b1=b1, b2=b2, eps=eps, wd=wd, clip=coef)
    ref_norm = g.float().norm()
    _close(gnorm, ref_norm.reshape(1), atol=1e-2, rtol=1e-4)
    scale = min(1.0, 1.0 / (ref_norm.item() + 1e-6))
    optim.adamw_ref(pr, mr, vr, g, lr=lr, b1=b1, b2=b2, eps=eps, wd=wd, step=step, grad_scale=scale)
    _close(p, pr, atol=1e-5, rtol=1e-4)
    _close(m, mr, atol=1e-6, rtol=1e-4)
    _close(v, vr, atol=1e-7, rtol=1e-4)
    _close(lowp, pr, atol=1e-2, rtol=1e-2)


def test_moe_route_permute_combine():
    T, E, k, H = 1000, 16, 4, 256
    logits = torch.randn(T, E, device=DEV)
    idx, w, counts, scores = moe.router_topk_cuda(logits, k)
    idx_r, w_r, counts_r = moe.route_topk(logits.cpu(), k)
    assert torch.equal(idx.cpu().sort(-1).values, idx_r.sort(-1).values)
    assert torch.equal(counts.cpu(), counts_r)
    _close(w.cpu().sort(-1).values, w_r.sort(-1).values, atol=1e-5, rtol=1e-4)
    _close(scores.cpu(), torch.softmax(logits.cpu(), -1), atol=1e-5, rtol=1e-4)

    for det in (False, True):
        plan = moe.build_plan(idx, counts, E, deterministic=det)
        x = _rand(T, H).requires_grad_()
        wt = w.clone().requires_grad_()
        xp = moe.permute(x, plan)
        total = int(plan.total_rows.item())
        assert total == int(((counts + 127) // 128 * 128).sum())
        # every pair lands on a row that belongs to its expert and holds its token
        slot = plan.slot.long()
        offs = plan.expert_offset.long()
        assert bool(((slot >= offs[idx.long()]) & (slot < offs[idx.long() + 1])).all())
        assert torch.equal(xp[slot[:, 0]], x.detach())
        rs = plan.row_src[:total]
        assert bool((xp[:total][rs < 0] == 0).all())
        be = plan.block_expert.cpu()
        for b in range(total // 128):
            assert offs[be[b]] <= b * 128 < offs[be[b] + 1]
        assert bool((be[total // 128:] == -1).all())
        y = moe.combine(xp * 1.0, wt, plan, T)
        dy = _rand(T, H)
        y.backward(dy)
        xr = x.detach().float().requires_grad_()
        wr = w.detach().clone().requires_grad_()
        yr = (xr[:, None, :] * wr[:, :, None]).sum(1)
        yr.backward(dy.float())
        _close(y, yr, atol=3e-2, rtol=2e-2)
        _close(x.grad, xr.grad, atol=5e-2, rtol=3e-2)
        _close(wt.grad, wr.grad, atol=0.3, rtol=3e-2)


def _blocks(counts):
    padded = (counts + 127) // 128 * 128
    offs = torch.zeros(len(counts) + 1, dtype=torch.int32)
    offs[1:] = padded.cumsum(0)
    P = int(offs[-1]) + 128
    be = torch.full((P // 128,), -1, dtype=torch.int32)
    for e in range(len(counts)):
        be[int(offs[e]) // 128:int(offs[e + 1]) // 128] = e
    return offs, be, P


def test_gemm_kgrouped():
    from prime_rl_b200.ops import lora
    counts = torch.tensor([130, 0, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    a, b = _rand(P, 200), _rand(P, 320)
    out = lora.kgrouped_gemm(a, b, offs.to(DEV), 4, alpha=0.5)
    rt.check_status()
    ref = lora.kgrouped_gemm(a.cpu(), b.cpu(), offs, 4, alpha=0.5)
    _close(out.cpu(), ref, atol=0.3, rtol=2e-2)
    assert bool((out[1] == 0).all())


def test_gemm_extra_reduction_segment():
    """C = A B^T + A2 B2^T in one pass (dense and grouped, K-major and MN-major B)."""
    from prime_rl_b200.ops.matmul import gemm, grouped_gemm_ref
    M, N, K, K2 = 300, 520, 200, 48
    a, b, a2, b2 = _rand(M, K), _rand(N, K), _rand(M, K2), _rand(N, K2)
    out = gemm(a, b, ext=(a2, b2))
    rt.check_status()
    ref = a.float() @ b.float().t() + a2.float() @ b2.float().t()
    _close(out, ref, atol=0.3, rtol=2e-2)
    # MN-major B (the input-gradient form): B [K, N], B2 [K2, N]
    bt, b2t = _rand(K, N), _rand(K2, N)
    out = gemm(a, bt, b_mn=True, ext=(a2, b2t))
    rt.check_status()
    _close(out, a.float() @ bt.float() + a2.float() @ b2t.float(), atol=0.3, rtol=2e-2)
    # grouped
    counts = torch.tensor([130, 0, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    E = 4
    x, t = _rand(P, K), _rand(P, K2)
    w, w2 = _rand(E, N, K), _rand(E, N, K2)
    out = gemm(x, w, block_expert=be.to(DEV), ext=(t, w2))
    rt.check_status()
    ref = grouped_gemm_ref(x.cpu(), w.cpu(), be, out_dtype=torch.float32) + \
        grouped_gemm_ref(t.cpu(), w2.cpu(), be, out_dtype=torch.float32)
    used = (be >= 0).repeat_interleave(128)
    _close(out.cpu()[used], ref[used], atol=0.3, rtol=2e-2)
    wt, w2t = _rand(E, K, N), _rand(E, K2, N)
    out = gemm(x, wt, b_mn=True, block_expert=be.to(DEV), ext=(t, w2t))
    rt.check_status()
    ref = grouped_gemm_ref(x.cpu(), wt.cpu(), be, b_mn=True, out_dtype=torch.float32) + \
        grouped_gemm_ref(t.cpu(), w2t.cpu(), be, b_mn=True, out_dtype=torch.float32)
    _close(out.cpu()[used], ref[used], atol=0.3, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("ranks,rank", [(1, 0), (2, 0), (2, 1), (4, 2)])
def test_gemm_with_all_gather_prologue_single_device(ranks, rank):
    """The all-gather GEMM with every "peer" buffer on this GPU: one kernel copies the other
    ranks' weight rows into the local buffer and multiplies, so the arrival counters, the rotated
    tile order and the async-proxy fence are exercised without a second GPU."""
    import ctypes

    torch.manual_seed(3)
    dev = torch.device("cuda")
    M, K, rows = 777, 328, 256
    N = rows * ranks
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
    bufs = []
    for r in range(ranks):                       # buffer of rank r: only its own rows are valid
        b = torch.full((N, K), float("nan"), device=dev, dtype=torch.bfloat16)
        b[r * rows:(r + 1) * rows] = w[r * rows:(r + 1) * rows]
        bufs.append(b)
    ptrs = (ctypes.c_void_p * ranks)(*[b.data_ptr() for b in bufs])
    ready = torch.zeros(N // 256, dtype=torch.int32, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    lib = rt.lib()
    for call in (1, 2):
        if call == 2:                            # counters keep growing across calls
            bufs[rank].fill_(float("nan"))
            bufs[rank][rank * rows:(rank + 1) * rows] = w[rank * rows:(rank + 1) * rows]
        rt.check(lib.prb_gemm_bf16_allgather(x.data_ptr(), bufs[rank].data_ptr(), ptrs, out.data_ptr(), M, N, K,
                                             x.stride(0), out.stride(0), 0, 0, 1.0, rank, ranks, rows,
                                             ready.data_ptr(), call, rt.status_tensor(dev).data_ptr(),
                                             rt.stream_ptr(dev)), "prb_gemm_bf16_allgather")
        torch.cuda.synchronize()
        rt.check_status()
        assert torch.equal(bufs[rank], w)
        ref = x.float() @ w.float().t()
        assert float((out.float() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_fp8_block_scaled_gemm_dense_and_grouped():
    """e4m3 operands with 1 x 128 / 128 x 128 scales against dequantise-then-multiply in fp32."""
    from prime_rl_b200.models.fp8 import quantize_to_fp8_blockwise
    from prime_rl_b200.ops import fp8
    M, N, K = 300, 520, 400
    x = _rand(M, K)
    w = _rand(N, K)
    xq, xs = fp8.quantize_act(x)
    xq_r, xs_r = fp8.quantize_act(x.cpu())
    assert torch.allclose(xs.cpu(), xs_r, rtol=1e-6)
    assert (xq.cpu().view(torch.float8_e4m3fn).float() - xq_r.view(torch.float8_e4m3fn).float()).abs().max() <= 32
    wq, ws = quantize_to_fp8_blockwise(w)
    out = fp8.fp8_gemm(xq, xs, wq.view(torch.uint8), ws)
    rt.check_status()
    ref = fp8.fp8_gemm_ref(xq, xs, wq, ws)
    _close(out, ref, atol=0.3, rtol=2e-2)
    # the quantised product stays close to the bf16 one
    full = x.float() @ w.float().t()
    assert ((out.float() - full).norm() / full.norm()) < 0.08
    # grouped
    counts = torch.tensor([130, 0, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    E = 4
    xp = _rand(P, K)
    wg = _rand(E, N, K)
    xpq, xps = fp8.quantize_act(xp)
    wgq, wgs = quantize_to_fp8_blockwise(wg)
    out = fp8.fp8_gemm(xpq, xps, wgq.view(torch.uint8), wgs, block_expert=be.to(DEV))
    rt.check_status()
    ref = fp8.fp8_gemm_ref(xpq.cpu(), xps.cpu(), wgq.cpu(), wgs.cpu(), be)
    used = (be >= 0).repeat_interleave(128)
    _close(out.cpu()[used], ref[used], atol=0.3, rtol=2e-2)


def test_lora_linear_and_grouped():
    from prime_rl_b200.ops import lora
    T, IN, r = 300, 256, 16
    segs = [384, 128, 128]
    x = _rand(T, IN).requires_grad_()
    w = _rand(sum(segs), IN, scale=0.05)
    a = _rand(len(segs) * r, IN, scale=0.1).requires_grad_()
    bs = [_rand(s, r, scale=0.1).requires_grad_() for s in segs]
    y = lora.lora_linear(x, w, a, bs, 2.0)
    dy = _rand(T, sum(segs))
    y.backward(dy)
    rt.check_status()
    xr, ar = x.detach().float().requires_grad_(), a.detach().float().requires_grad_()
    bsr = [b.detach().float().requires_grad_() for b in bs]
    yr = lora.lora_linear_ref(xr, w.float(), ar, bsr, 2.0)
    yr.backward(dy.float())
    _close(y, yr, atol=0.1, rtol=2e-2)
    _close(x.grad, xr.grad, atol=0.1, rtol=3e-2)
    _close(a.grad, ar.grad, atol=0.5, rtol=3e-2)
    for b, br in zip(bs, bsr):
        _close(b.grad, br.grad, atol=0.5, rtol=3e-2)

    # grouped (experts)
    E, H, I = 4, 256, 128
    counts = torch.tensor([130, 0, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    xp = _rand(P, H)
    used = int(offs[-1])
    xp[used:] = 0
    xp.requires_grad_()
    wg = _rand(E, 2 * I, H, scale=0.05)
    ag = _rand(E, 2 * r, H, scale=0.1).requires_grad_()
    bg = [_rand(E, I, r, scale=0.1).requires_grad_() for _ in range(2)]
    yg = lora.lora_grouped_linear(xp, wg, ag, bg, 2.0, be.to(DEV), offs.to(DEV))
    dyg = _rand(P, 2 * I)
    dyg[used:] = 0
    yg.backward(dyg)
    rt.check_status()
    xc = xp.detach().cpu().float().requires_grad_()
    agc = ag.detach().cpu().float().requires_grad_()
    bgc = [b.detach().cpu().float().requires_grad_() for b in bg]
    ygc = lora.lora_grouped_linear(xc, wg.cpu().float(), agc, bgc, 2.0, be, offs)
    ygc.backward(dyg.cpu().float())
    _close(yg[:used].cpu(), ygc[:used], atol=0.1, rtol=3e-2)
    _close(xp.grad[:used].cpu(), xc.grad[:used], atol=0.1, rtol=3e-2)
    _close(ag.grad.cpu(), agc.grad, atol=0.5, rtol=3e-2)
    for b, bc in zip(bg, bgc):
        _close(b.grad.cpu(), bc.grad, atol=0.5, rtol=3e-2)


def test_qkv_norm_rope_packed_projection():
    T, nq, nkv, D = 300, 4, 2, 128
    W = (nq + 2 * nkv) * D
    qkv = _rand(T, W).requires_grad_()
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    pos = torch.randint(0, 4096, (T,), device=DEV, dtype=torch.int32)
    inv_f = rope.inv_freq(D, 1e6, device=DEV)
    q, k, v = rope.qkv_norm_rope(qkv, qw, kw, pos, inv_f, 1e-6, nq, nkv, D)
    gq, gk, gv = _rand(T, nq, D), _rand(T, nkv, D), _rand(T, nkv, D)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    ref = qkv.detach().float().requires_grad_()
    qwr, kwr = qw.detach().float().requires_grad_(), kw.detach().float().requires_grad_()
    qd, kd = nq * D, nkv * D
    qr = rope.qknorm_rope_ref(ref[:, :qd].view(T, nq, D), qwr, pos, inv_f, 1e-6)
    kr = rope.qknorm_rope_ref(ref[:, qd:qd + kd].view(T, nkv, D), kwr, pos, inv_f, 1e-6)
    vr = ref[:, qd + kd:].view(T, nkv, D)
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    _close(q, qr, atol=3e-2, rtol=2e-2)
    _close(k, kr, atol=3e-2, rtol=2e-2)
    _close(v, vr, atol=1e-6, rtol=0)
    _close(qkv.grad, ref.grad, atol=6e-2, rtol=3e-2)
    _close(qw.grad, qwr.grad, atol=1.0, rtol=3e-2)
    # the non-contiguous single-tensor path must also honour the pitches
    qs = qkv.detach()[:, :qd].view(T, nq, D).requires_grad_()
    y = rope.qknorm_rope(qs, qw.detach(), pos, inv_f, 1e-6)
    y.backward(gq)
    assert qs.grad.shape == (T, nq, D)


@pytest.mark.parametrize("lens,window", [([256], None), ([300, 77, 1000], None), ([5, 640, 129], None),
                                         ([700, 300], 200), ([2048], None)])
def test_flash_fwd_matches_reference(lens, window):
    from prime_rl_b200.ops import attention as A, flash_native
    T, Hq, Hkv, D = sum(lens), 8, 2, 128
    q, k, v = _rand(T, Hq, D), _rand(T, Hkv, D), _rand(T, Hkv, D)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.to(DEV)
    out, lse = flash_native.flash_fwd(q, k, v, cu, window=window)
    rt.check_status()
    ref = A.attention_ref(q, k, v, cu, window=window)
    _close(out, ref, atol=2e-2, rtol=2e-2)
    # lse against an fp32 computation
    scale = D ** -0.5
    kk = k.float().repeat_interleave(Hq // Hkv, 1)
    s = torch.einsum("thd,shd->hts", q.float(), kk) * scale
    pos = torch.arange(T, device=DEV)
    doc = torch.searchsorted(cu[1:].long().contiguous(), pos, right=True)
    mask = (doc[:, None] == doc[None, :]) & (pos[None, :] <= pos[:, None])
    if window is not None:
        mask &= pos[:, None] - pos[None, :] < window
    ref_lse = torch.logsumexp(s.masked_fill(~mask[None], float("-inf")), dim=-1)
    _close(lse, ref_lse, atol=1e-2, rtol=1e-3)


def test_flash_attention_autograd_and_cache():
    from prime_rl_b200.ops import attention as A
    lens = [300, 212]
    T, Hq, Hkv, D = sum(lens), 4, 2, 128
    q, k, v = (_rand(T, Hq, D).requires_grad_(), _rand(T, Hkv, D).requires_grad_(), _rand(T, Hkv, D).requires_grad_())
    cu = torch.tensor([0, 300, 512], dtype=torch.int32, device=DEV)
    cache = {}
    with torch.no_grad():
        o1 = A.attention(q, k, v, cu, 300, cache=cache, cache_key=0)
    assert 0 in cache
    launches = rt.launch_count()
    o2 = A.attention(q, k, v, cu, 300, cache=cache, cache_key=0)
    assert rt.launch_count() == launches and 0 not in cache    # reused, nothing launched
    assert torch.equal(o1, o2)
    do = _rand(T, Hq, D)
    o2.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    A.attention_ref(qr, kr, vr, cu).backward(do.float())
    _close(q.grad, qr.grad, atol=5e-2, rtol=5e-2)
    _close(k.grad, kr.grad, atol=5e-2, rtol=5e-2)
    _close(v.grad, vr.grad, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("lens,window", [([128], None), ([256], None), ([300, 77, 1000], None), ([700, 300], 200)])
def test_flash_bwd_matches_reference(lens, window):
    from prime_rl_b200.ops import attention as A, flash_native
    T, Hq, Hkv, D = sum(lens), 4, 2, 128
    q, k, v = _rand(T, Hq, D), _rand(T, Hkv, D), _rand(T, Hkv, D)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.to(DEV)
    out, lse = flash_native.flash_fwd(q, k, v, cu, window=window)
    do = _rand(T, Hq, D)
    dq, dk, dv = flash_native.flash_bwd(do, q, k, v, out, lse, cu, window=window)
    rt.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    A.attention_ref(qr, kr, vr, cu, window=window).backward(do.float())
    for got, want, name in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
        rel = (got.float() - want).norm() / want.norm()
        assert rel < 2e-2, f"{name}: relative error {rel:.4f}"
        _close(got, want, atol=0.1, rtol=5e-2)


@pytest.mark.parametrize("lens,window,cp", [([300, 77, 1000], None, 3), ([700, 300], 200, 2), ([1024], None, 4)])
def test_flash_query_slices_sum_to_full_attention(lens, window, cp):
    """Context-parallel form: each slice of the query rows against all keys reproduces its rows of
    the full attention, and the per-slice dK / dV add up to the full gradients."""
    from prime_rl_b200.ops import attention as A, flash_native
    T, Hq, Hkv, D = sum(lens), 4, 2, 128
    pad = (-T) % cp
    lens = lens[:-1] + [lens[-1] + pad]
    T += pad
    q, k, v = _rand(T, Hq, D), _rand(T, Hkv, D), _rand(T, Hkv, D)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.to(DEV)
    do = _rand(T, Hq, D)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, cu, window=window)
    ref.backward(do.float())
    Tl = T // cp
    dk_sum = torch.zeros(T, Hkv, D, device=DEV)
    dv_sum = torch.zeros(T, Hkv, D, device=DEV)
    for r in range(cp):
        lo = r * Tl
        ql, dol = q[lo:lo + Tl].contiguous(), do[lo:lo + Tl].contiguous()
        out, lse = flash_native.flash_fwd(ql, k, v, cu, window=window, q_offset=lo)
        dq, dk, dv = flash_native.flash_bwd(dol, ql, k, v, out, lse, cu, window=window, q_offset=lo)
        rt.check_status()
        _close(out, ref[lo:lo + Tl], atol=3e-2, rtol=3e-2)
        rel = (dq.float() - qr.grad[lo:lo + Tl]).norm() / qr.grad[lo:lo + Tl].norm()
        assert rel < 2e-2, f"dq slice {r}: relative error {rel:.4f}"
        dk_sum += dk.float()
        dv_sum += dv.float()
    for got, want, name in ((dk_sum, kr.grad, "dk"), (dv_sum, vr.grad, "dv")):
        rel = (got - want).norm() / want.norm()
        assert rel < 2e-2, f"{name}: relative error {rel:.4f}"


@pytest.mark.parametrize("lens,window,chunks", [([1024], None, 4), ([300, 77, 1000, 159], None, 4), ([700, 300, 200], 200, 6),
                                                 ([2048], None, 8), ([130, 126], None, 2)])
def test_flash_key_blocks_merge_to_full_attention(lens, window, chunks):
    """Ring form of context parallelism on one device: every (query chunk, key chunk) block computed on its own
    (chunk edges fall inside 128-row tiles and inside documents), partial results merged through the log-sum-exp
    give the full attention; block gradients taken with the final output / log-sum-exp add up to the full ones."""
    from prime_rl_b200.ops import attention as A, flash_native
    from prime_rl_b200.parallel import ring_attn
    T, Hq, Hkv, D = sum(lens), 4, 2, 128
    assert T % chunks == 0
    c = T // chunks
    q, k, v = _rand(T, Hq, D), _rand(T, Hkv, D), _rand(T, Hkv, D)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    cu = cu.to(DEV)
    do = _rand(T, Hq, D)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, cu, window=window)
    ref.backward(do.float())

    acc = torch.zeros(T, Hq, D, device=DEV)
    lse = torch.empty(Hq, T, device=DEV)
    for qi in range(chunks):
        rows = slice(qi * c, (qi + 1) * c)
        a = acc[rows]
        l = torch.full((Hq, c), float("-inf"), device=DEV)
        for ki in range(chunks):            # blocks above the diagonal come back empty and leave the rows unchanged
            keys = slice(ki * c, (ki + 1) * c)
            part, lp = flash_native.flash_fwd_block(q[rows], k[keys], v[keys], cu, T, qi * c, ki * c, window=window)
            if ki > qi:
                assert torch.isinf(lp).all() and float(part.float().abs().max()) == 0.0
            else:
                want, want_lse, _ = ring_attn.block_fwd_ref(q[rows], k[keys], v[keys], cu.long(), T, qi * c, ki * c, window)
                seen = ~torch.isinf(want_lse)
                assert torch.equal(seen, ~torch.isinf(lp))
                _close(lp[seen], want_lse[seen], atol=2e-2, rtol=2e-2)
                _close(part, want, atol=3e-2, rtol=3e-2)
            ring_attn.merge_partial(a, l, part, lp)
        lse[:, rows] = l
    rt.check_status()
    _close(acc, ref, atol=3e-2, rtol=3e-2)
    full_out, full_lse = flash_native.flash_fwd(q, k, v, cu, window=window)
    _close(lse, full_lse, atol=2e-2, rtol=2e-2)

    out = acc.to(torch.bfloat16)
    dq = torch.zeros(T, Hq, D, device=DEV)
    dk = torch.zeros(T, Hkv, D, device=DEV)
    dv = torch.zeros(T, Hkv, D, device=DEV)
    for qi in range(chunks):
        rows = slice(qi * c, (qi + 1) * c)
        for ki in range(qi + 1):
            keys = slice(ki * c, (ki + 1) * c)
            a, b, e = flash_native.flash_bwd_block(do[rows], q[rows], k[keys], v[keys], out[rows],
                                                   lse[:, rows].contiguous(), cu, T, qi * c, ki * c, window=window)
            dq[rows] += a.float()
            dk[keys] += b.float()
            dv[keys] += e.float()
    rt.check_status()
    for got, want, name in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
        rel = (got - want).norm() / want.norm()
        assert rel < 2e-2, f"{name}: relative error {rel:.4f}"


@pytest.mark.parametrize("Hq,Hkv", [(32, 4), (8, 8), (16, 4)])
@pytest.mark.parametrize("splits", [1, 3])
def test_paged_decode(Hq, Hkv, splits):
    from prime_rl_b200.ops import paged
    B, D, ps, pages = 5, 128, 16, 64
    kpool, vpool = _rand(pages, ps, Hkv, D), _rand(pages, ps, Hkv, D)
    ctx = torch.tensor([1, 17, 250, 64, 300], dtype=torch.int32)
    perm = torch.randperm(pages)
    bt = torch.zeros(B, 20, dtype=torch.int32)
    used = 0
    for b in range(B):
        n = (int(ctx[b]) + ps - 1) // ps
        bt[b, :n] = perm[used:used + n] if used + n <= pages else perm[:n]
        used = (used + n) % (pages - 20)
    q = _rand(B, Hq, D)
    out = paged.paged_decode_raw(q, kpool, vpool, bt.to(DEV), ctx.to(DEV), splits=splits)
    ref = paged.paged_decode_ref(q, kpool, vpool, bt.to(DEV), ctx)
    _close(out, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("H,topk", [(128, 128), (64, 192), (16, 64)])
def test_sparse_mla_forward_kernel_and_recomputed_backward(H, topk):
    from prime_rl_b200.ops import sparse_mla

    torch.manual_seed(11)
    dev = torch.device("cuda")
    T, S = 150, 700
    q = (torch.randn(T, H, 576, device=dev) * 0.5).bfloat16().requires_grad_()
    kv = (torch.randn(S, 576, device=dev) * 0.5).bfloat16().requires_grad_()
    idx = torch.stack([torch.randperm(S, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
    idx[:, topk // 2:][torch.rand(T, topk - topk // 2, device=dev) < 0.4] = S      # empty slots
    idx[3] = S                                                                      # a query without any slot
    idx[7, : topk - 1] = S                                                          # exactly one slot, in the last block
    scale = 576 ** -0.5
    out = sparse_mla.sparse_mla_attention(q, kv, idx, scale, 512)
    torch.cuda.synchronize()
    rt.check_status()
    qf, kvf = q.detach().float().requires_grad_(), kv.detach().float().requires_grad_()
    ref = sparse_mla.sparse_mla_attention_ref(qf, kvf, idx, scale, 512)
    assert out.shape == (T, H, 512) and float(out[3].abs().max()) == 0.0
    err = float((out.float() - ref).abs().max())
    assert err < 2e-2, err
    dout = torch.randn_like(out)
    out.backward(dout)
    ref.backward(dout.float())
    for a, b in ((q.grad, qf.grad), (kv.grad, kvf.grad)):
        rel = float((a.float() - b).norm() / b.norm())
        assert rel < 3e-2, rel


@pytest.mark.gpu
@pytest.mark.parametrize("cp,rank", [(2, 1), (4, 2), (2, 0)])
def test_flash_forward_with_in_kernel_kv_gather_single_device(cp, rank):
    """The context-parallel forward whose gather warp pulls the lower ranks' K / V chunks itself,
    with every "peer" buffer on this GPU (one kernel, no cross-launch waits): the result equals
    the query-slice kernel on complete K / V, and the local buffer ends up holding the chunks."""
    import ctypes

    from prime_rl_b200.ops import flash_native

    torch.manual_seed(21)
    dev = torch.device("cuda")
    Tl, Hq, Hkv, D = 640, 8, 2, 128
    T = Tl * cp
    lens = [T // 2 - 100, T // 2 + 100]
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device=dev)
    q = torch.randn(Tl, Hq, D, device=dev).bfloat16()
    k = torch.randn(T, Hkv, D, device=dev).bfloat16()
    v = torch.randn(T, Hkv, D, device=dev).bfloat16()
    bufs = []
    for r in range(cp):                       # rank r's buffer: [K | V], only its own chunk is valid
        b = torch.zeros(2, T, Hkv, D, device=dev, dtype=torch.bfloat16)
        b[0, r * Tl:(r + 1) * Tl] = k[r * Tl:(r + 1) * Tl]
        b[1, r * Tl:(r + 1) * Tl] = v[r * Tl:(r + 1) * Tl]
        bufs.append(b)
    ptrs = (ctypes.c_void_p * cp)(*[b.data_ptr() for b in bufs])
    counters = torch.zeros(cp + 1, dtype=torch.int32, device=dev)
    mine = bufs[rank]
    out, lse = flash_native.flash_fwd_gather(q, mine[0], mine[1], ptrs, cu, rank, cp, counters)
    torch.cuda.synchronize()
    rt.check_status()
    ref_out, ref_lse = flash_native.flash_fwd(q, k, v, cu, q_offset=rank * Tl)
    assert torch.equal(mine[0, : (rank + 1) * Tl], k[: (rank + 1) * Tl])
    assert torch.equal(mine[1, : (rank + 1) * Tl], v[: (rank + 1) * Tl])
    assert float((out.float() - ref_out.float()).abs().max()) < 1e-6
    assert float((lse - ref_lse).abs().max()) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("C,K,act,with_bias", [(264, 4, "silu", True), (64, 4, "silu", False), (40, 3, None, True)])
def test_causal_conv1d_kernel_forward_and_backward(C, K, act, with_bias):
    from prime_rl_b200.ops import ssm

    torch.manual_seed(31)
    dev = torch.device("cuda")
    lengths = [70, 1, 3, 129, 40]
    T = sum(lengths)
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(dev)
    x = torch.randn(T, C, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(C, K, device=dev) * 0.5).bfloat16().requires_grad_()
    b = torch.randn(C, device=dev).bfloat16().requires_grad_() if with_bias else None
    y = ssm.causal_conv1d(x, w, b, pos, act)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    bf = b.detach().float().requires_grad_() if with_bias else None
    ref = ssm.causal_conv1d_ref(xf, wf, bf, pos, act)
    assert float((y.float() - ref).abs().max()) < 3e-2
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    assert float((x.grad.float() - xf.grad).abs().max()) < 5e-2
    assert float((w.grad.float() - wf.grad).abs().max() / wf.grad.abs().max()) < 2e-2
    if with_bias:
        assert float((b.grad.float() - bf.grad).abs().max() / bf.grad.abs().max()) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,group,shared_w,gate_first", [(77, 1024, 128, False, True), (200, 2048, 1024, False, True),
                                                               (333, 128, 128, True, False), (50, 64, 64, True, False)])
def test_gated_group_rmsnorm_kernel(rows, cols, group, shared_w, gate_first):
    from prime_rl_b200.ops import ssm

    torch.manual_seed(41)
    dev = torch.device("cuda")
    x = torch.randn(rows, cols, device=dev).bfloat16().requires_grad_()
    g = torch.randn(rows, cols, device=dev).bfloat16().requires_grad_()
    w = (1 + 0.2 * torch.randn(group if shared_w else cols, device=dev)).bfloat16().requires_grad_()
    y = ssm.gated_rms_norm(x, g, w, 1e-5, group, "silu", gate_first)
    xf, gf, wf = (t.detach().float().requires_grad_() for t in (x, g, w))
    ref = ssm.gated_rms_norm_ref(xf, gf, wf, 1e-5, group, "silu", gate_first)
    assert float((y.float() - ref).abs().max()) < 4e-2
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    for a, b in ((x.grad, xf.grad), (g.grad, gf.grad), (w.grad, wf.grad)):
        assert float((a.float() - b).abs().max() / b.abs().max()) < 2e-2


def test_allreduce_add_rmsnorm_kernel_with_emulated_peers():
    """The tensor-parallel reduce kernel on one GPU: the "peers" are local buffers and the peer's flag
    slot is set beforehand, so the single launch waits on nothing. Two consecutive calls check the
    device-side call counter."""
    import ctypes

    from prime_rl_b200.ops import _runtime as rt

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    rows, cols, R = 300, 2048, 2
    parts = [torch.randn(rows, cols, device=dev).bfloat16() for _ in range(R)]
    res = torch.randn(rows, cols, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(cols, device=dev)).bfloat16()
    flags = [torch.zeros(R, dtype=torch.int32, device=dev) for _ in range(R)]
    flags[0][1] = 1 << 30                                     # "rank 1 has arrived", for every call to come
    pp = (ctypes.c_void_p * R)(*[p.data_ptr() for p in parts])
    fp = (ctypes.c_void_p * R)(*[f.data_ptr() for f in flags])
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    out_h, out_x = torch.empty_like(res), torch.empty_like(res)
    for call in (1, 2):
        rt.check(rt.lib().prb_ar_add_rmsnorm(pp, fp, state.data_ptr(), res.data_ptr(), w.data_ptr(), out_h.data_ptr(),
                                             out_x.data_ptr(), rows, cols, 1e-6, 0, R, rt.status_tensor(dev).data_ptr(),
                                             rt.stream_ptr(dev)), "prb_ar_add_rmsnorm")
        torch.cuda.synchronize()
        rt.check_status()
        assert state.tolist() == [call, 0]
        assert flags[0][0].item() == call and flags[1][0].item() == call     # announced to itself and to the peer
    h = parts[0].float() + parts[1].float() + res.float()
    torch.testing.assert_close(out_h.float(), h, atol=0.04, rtol=0.01)
    hb = out_h.float()
    ref = hb * torch.rsqrt(hb.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    torch.testing.assert_close(out_x.float(), ref, atol=0.03, rtol=0.01)
    # no residual, no norm output
    rt.check(rt.lib().prb_ar_add_rmsnorm(pp, fp, state.data_ptr(), None, None, out_h.data_ptr(), None, rows, cols, 1e-6, 0,
                                         R, rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)), "prb_ar_add_rmsnorm")
    torch.cuda.synchronize()
    torch.testing.assert_close(out_h.float(), parts[0].float() + parts[1].float(), atol=0.04, rtol=0.01)


def test_moe_inference_path_skips_padding_rows_and_matches_the_training_path():
    """Under no_grad the MoE layer leaves the rows that pad every expert to 128 untouched (no zero fill, no
    GLU, no GEMM stores); the tokens' outputs must be bit-identical to the regular path."""
    from prime_rl_b200.models import ModelArch, SeqInfo
    from prime_rl_b200.models.layers import MoE

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    arch = ModelArch(model_type="qwen3_moe", hidden_size=512, num_hidden_layers=1, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=128, intermediate_size=512, num_experts=16, num_experts_per_tok=4,
                     moe_intermediate_size=256, vocab_size=256)
    moe = MoE(arch, 0, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        for p in moe.parameters():
            p.normal_(0, 0.05)
    x = torch.randn(37, 512, device=dev).bfloat16()
    seq = SeqInfo(None, 0, torch.arange(37, dtype=torch.int32, device=dev))
    # poison the allocator's free blocks so that untouched padding rows hold NaNs
    junk = torch.full((64 * 128, 512), float("nan"), device=dev, dtype=torch.bfloat16)
    del junk
    with torch.no_grad():
        assert moe.experts.supports_row_mask(x)
        y_inf = moe(x, seq)
        moe.experts.supports_row_mask = lambda _x: False          # same arithmetic through the zero-padded path
        y_ref = moe(x, seq)
    assert torch.isfinite(y_inf.float()).all()
    assert torch.equal(y_inf, y_ref)


def test_fp8_experts_skip_padding_rows_and_match_the_padded_fp8_path():
    """fp8 expert weights at inference: token rows are quantised once and gathered as fp8, every kernel skips the
    rows that pad an expert to 128. Must agree with the zero-padded fp8 path (same quantised operands) and stay
    close to the bf16 result; padding rows poisoned with NaNs must not leak."""
    from prime_rl_b200.models import ModelArch, SeqInfo
    from prime_rl_b200.models.layers import MoE
    from prime_rl_b200.ops import fp8

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    arch = ModelArch(model_type="qwen3_moe", hidden_size=512, num_hidden_layers=1, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=128, intermediate_size=512, num_experts=16, num_experts_per_tok=4,
                     moe_intermediate_size=256, vocab_size=256)
    moe = MoE(arch, 0, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        for p in moe.parameters():
            p.normal_(0, 0.05)
    x = torch.randn(53, 512, device=dev).bfloat16()
    seq = SeqInfo(None, 0, torch.arange(53, dtype=torch.int32, device=dev))
    with torch.no_grad():
        y_bf16 = moe(x, seq)
        assert moe.experts.quantize_fp8_()
        junk = torch.full((64 * 128, 512), float("nan"), device=dev, dtype=torch.bfloat16)
        del junk
        assert moe.experts.supports_fp8_row_mask(x)
        y_masked = moe(x, seq)
        moe.experts.supports_fp8_row_mask = lambda _x: False      # zero-padded rows through the same fp8 GEMMs
        moe.experts.supports_row_mask = lambda _x: False
        y_padded = moe(x, seq)
    rt.check_status()
    assert torch.isfinite(y_masked.float()).all()
    _close(y_masked, y_padded, atol=2e-2, rtol=2e-2)
    assert ((y_masked.float() - y_bf16.float()).norm() / y_bf16.float().norm()) < 0.1
    # the masked quantiser leaves padding rows alone and agrees with the full one on the others
    h = torch.randn(256, 384, device=dev).bfloat16()
    valid = torch.full((256,), -1, dtype=torch.int32, device=dev)
    valid[::3] = 1
    q_all, s_all = fp8.quantize_act(h)
    q_m, s_m = fp8.quantize_act(h, row_valid=valid)
    assert torch.equal(q_m[::3], q_all[::3]) and torch.equal(s_m[::3], s_all[::3])


def test_qkv_rope_to_cache_matches_separate_ops():
    """Fused split + QK-norm + rotary + paged-cache write against qkv_norm_rope followed by index_copy_
    (bit-equal), with and without the contiguous K / V outputs and without QK-norm."""
    from prime_rl_b200 import ops

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    T, nq, nkv, D, pages, ps = 77, 8, 2, 128, 12, 16
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=dev).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device=dev)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, device=dev)).bfloat16()
    pos = torch.randint(0, 4000, (T,), device=dev, dtype=torch.int32)
    inv_f = ops.inv_freq(D, 1e6, device=dev)
    slots = torch.randperm(pages * ps, device=dev)[:T]
    for norm in (True, False):
        a, b = (qw, kw) if norm else (None, None)
        with torch.no_grad():
            q0, k0, v0 = ops.qkv_norm_rope(qkv, a, b, pos, inv_f, 1e-6, nq, nkv, D)
            kc0 = torch.zeros(pages, ps, nkv, D, device=dev, dtype=torch.bfloat16)
            vc0 = torch.zeros_like(kc0)
            kc0.view(-1, nkv, D).index_copy_(0, slots, k0)
            vc0.view(-1, nkv, D).index_copy_(0, slots, v0)
            for want in (True, False):
                kc, vc = torch.zeros_like(kc0), torch.zeros_like(vc0)
                q, k, v = ops.qkv_rope_to_cache(qkv, a, b, pos, inv_f, 1e-6, nq, nkv, D, kc, vc, slots, want_kv=want)
                assert torch.equal(q, q0) and torch.equal(kc, kc0) and torch.equal(vc, vc0)
                if want:
                    assert torch.equal(k, k0) and torch.equal(v, v0)
                else:
                    assert k is None and v is None


def test_allreduce_kernel_wait_runs_out_when_the_peer_never_arrives():
    """The peer's flag slot stays 0: the bounded wait of the tensor-parallel reduce gives up (about 2 s of GPU
    time), records kTimeoutPeerFlag, writes nothing, still advances its call counter and returns; the device
    keeps answering. This is what a rank sees when its peer has left between two steps."""
    import ctypes

    from prime_rl_b200.ops import _runtime as rt

    dev = torch.device("cuda", 0)
    rows, cols, R = 4, 256, 2
    parts = [torch.ones(rows, cols, device=dev).bfloat16() for _ in range(R)]
    flags = [torch.zeros(R, dtype=torch.int32, device=dev) for _ in range(R)]
    pp = (ctypes.c_void_p * R)(*[p.data_ptr() for p in parts])
    fp = (ctypes.c_void_p * R)(*[f.data_ptr() for f in flags])
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    out_h = torch.full((rows, cols), 7.0, device=dev).bfloat16()
    st = rt.status_tensor(dev)
    st.zero_()
    rc = rt.lib().prb_ar_add_rmsnorm(pp, fp, state.data_ptr(), None, None, out_h.data_ptr(), None, rows, cols, 1e-6, 0, R,
                                     st.data_ptr(), rt.stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 5            # kTimeoutPeerFlag
    with pytest.raises(Exception):
        rt.check_status()
    st.zero_()
    assert float(out_h.float().min()) == 7.0 and state.tolist() == [1, 0]
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0      # the device still answers


def test_route_and_plan_small_matches_the_separate_kernels():
    """One-launch router + plan for decode batches against router_topk + build_plan: same experts, weights,
    histogram, offsets and block table; slots form a valid placement (row_src inverts slot, rows stay inside
    their expert's range, everything else is padding)."""
    from prime_rl_b200.ops import moe as moe_ops

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    moe_ops.SMALL_ROUTE_TOKENS, keep = 1024, moe_ops.SMALL_ROUTE_TOKENS     # exercise several tokens per warp too
    for T, E, k, func, bias in ((256, 128, 8, "softmax", False), (37, 64, 6, "sigmoid", True), (1, 16, 2, "softmax", False)):
        logits = torch.randn(T, E, device=dev)
        sel_bias = torch.randn(E, device=dev) * 0.1 if bias else None
        with torch.no_grad():
            fused = moe_ops.route_and_plan_small(logits, k, score_func=func, norm_topk=True, route_scale=1.5, sel_bias=sel_bias)
            assert fused is not None
            idx, w, counts, plan = fused
            idx0, w0, counts0 = moe_ops.route_topk(logits, k, score_func=func, norm_topk=True, route_scale=1.5, sel_bias=sel_bias)
            plan0 = moe_ops.build_plan(idx0, counts0, E)
        assert torch.equal(idx, idx0) and torch.equal(w, w0) and torch.equal(counts, counts0)
        assert torch.equal(plan.expert_offset, plan0.expert_offset) and torch.equal(plan.block_expert, plan0.block_expert)
        assert torch.equal(plan.total_rows, plan0.total_rows) and plan.max_rows == plan0.max_rows
        slot, row_src = plan.slot.reshape(-1).long(), plan.row_src
        assert torch.equal(row_src[slot], torch.arange(T * k, device=dev, dtype=torch.int32))
        assert int((row_src >= 0).sum()) == T * k
        off = plan.expert_offset.long()
        e = idx.reshape(-1).long()
        assert bool(((slot >= off[e]) & (slot < off[e] + counts.long()[e])).all())
    moe_ops.SMALL_ROUTE_TOKENS = keep
    with torch.enable_grad():
        assert moe_ops.route_and_plan_small(torch.randn(4, 16, device=dev), 2) is None
    with torch.no_grad():
        assert moe_ops.route_and_plan_small(torch.randn(keep + 1, 16, device=dev), 2) is None


def test_weight_gradients_accumulate_straight_into_the_fp32_buffer():
    """With a gradient accumulator attached to the weight, the dense and the grouped weight-gradient GEMMs add
    into it (fp32, beta = 1) and hand autograd no gradient; two backward passes must equal the sum of the two
    ordinary bf16 gradients."""
    from prime_rl_b200.ops import matmul as mm

    torch.manual_seed(0)
    x = _rand(300, 256).requires_grad_()
    w = torch.nn.Parameter(_rand(384, 256, scale=0.05))
    dy = _rand(300, 384)
    mm.linear(x, w).backward(dy)
    ref = w.grad.float().clone()
    w.grad = None
    w._grad_acc = torch.zeros(384, 256, dtype=torch.float32, device=DEV)
    for _ in range(2):
        mm.linear(x, w).backward(dy)
    rt.check_status()
    assert w.grad is None
    _close(w._grad_acc, 2 * ref, atol=0.05, rtol=2e-2)
    # grouped: experts with and without rows
    counts = torch.tensor([130, 0, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    xg = _rand(P, 128)
    valid = (be >= 0).repeat_interleave(128).to(DEV)
    xg = (xg * valid[:, None]).requires_grad_()
    wg = torch.nn.Parameter(_rand(4, 192, 128, scale=0.05))
    dyg = _rand(P, 192) * valid[:, None]
    mm.grouped_linear(xg, wg, be.to(DEV), offs.to(DEV)).backward(dyg)
    refg = wg.grad.float().clone()
    wg.grad = None
    wg._grad_acc = torch.full((4, 192, 128), 1.0, dtype=torch.float32, device=DEV)
    mm.grouped_linear(xg, wg, be.to(DEV), offs.to(DEV)).backward(dyg)
    rt.check_status()
    assert wg.grad is None
    _close(wg._grad_acc, refg + 1.0, atol=0.05, rtol=2e-2)
    assert torch.equal(wg._grad_acc[1], torch.ones(192, 128, device=DEV))      # an expert without rows adds nothing


@pytest.mark.parametrize("Hq,Hkv", [(32, 4), (8, 2), (8, 8)])
def test_paged_decode_with_shared_prefix_groups_matches_the_reference(Hq, Hkv):
    """Sequences whose leading pages are the same physical pages are attended in two passes (shared pages once per
    group of up to 8 sequences, own pages per sequence) and merged: must equal the plain per-sequence result.
    Covers full groups, a group of 3, a sequence in no group, and a shared run that is not a multiple of the
    kernel's four-page stage."""
    from prime_rl_b200.ops import paged

    torch.manual_seed(0)
    D, ps, n_pages = 128, 16, 400
    kpool = _rand(n_pages, ps, Hkv, D)
    vpool = _rand(n_pages, ps, Hkv, D)
    free = list(range(n_pages))
    import random

    random.Random(0).shuffle(free)
    page_lists, lengths = [], []

    def family(n_members, shared_pages, own_tokens):
        shared = [free.pop() for _ in range(shared_pages)]
        for i in range(n_members):
            n_own = own_tokens[i]
            own = [free.pop() for _ in range((n_own + ps - 1) // ps)]
            page_lists.append(shared + own)
            lengths.append(shared_pages * ps + n_own)

    family(8, 9, [1, 5, 16, 17, 33, 2, 40, 9])        # 9 shared pages: 2 full stages + 1 page
    family(3, 4, [3, 20, 1])
    family(1, 6, [7])                                   # alone: no group
    family(8, 5, [12] * 8)
    B = len(page_lists)
    W = max(len(p) for p in page_lists)
    bt = torch.zeros(B, W, dtype=torch.int32)
    for i, p in enumerate(page_lists):
        bt[i, :len(p)] = torch.tensor(p, dtype=torch.int32)
    ctx = torch.tensor(lengths, dtype=torch.int32)
    q = _rand(B, Hq, D)
    ref = paged.paged_decode_ref(q.cpu(), kpool.cpu(), vpool.cpu(), bt, ctx).to(DEV)
    # kv.length of the runner is the length before the new token: the last key of a sequence is its own
    groups, page_begin = paged.group_shared_prefixes(page_lists, [n - 1 for n in lengths], ps, min_pages=4)
    assert sorted(len(m) for m, _ in groups) == [3, 8, 8] and page_begin[11] == 0
    n_slots = B // 2
    gs = torch.full((n_slots, 8), -1, dtype=torch.int32)
    gp = torch.zeros(n_slots, dtype=torch.int32)
    for gi, (members, shared) in enumerate(groups):
        gs[gi, :len(members)] = torch.tensor(members, dtype=torch.int32)
        gp[gi] = shared
    pb = torch.tensor(page_begin, dtype=torch.int32)
    for splits, psplits in ((1, 1), (2, 2), (3, 4)):
        out = paged.paged_decode_raw(q, kpool, vpool, bt.to(DEV), ctx.to(DEV), splits=splits,
                                     prefix=(pb.to(DEV), gs.to(DEV), gp.to(DEV), psplits))
        _close(out, ref, atol=2e-2, rtol=2e-2)
    # no groups at all: the prefix slots must be ignored
    out = paged.paged_decode_raw(q, kpool, vpool, bt.to(DEV), ctx.to(DEV), splits=2,
                                 prefix=(torch.zeros_like(pb).to(DEV), torch.full_like(gs, -1).to(DEV),
                                         torch.zeros_like(gp).to(DEV), 2))
    _close(out, ref, atol=2e-2, rtol=2e-2)


def test_multi_adapter_lora_linear_and_experts_match_the_reference_path():
    """Several adapters in one launch (masked rank columns inside the base GEMM's extra reduction segment) against
    the per-adapter PyTorch composition, forward and gradients, dense and grouped."""
    from prime_rl_b200.ops import lora as L

    torch.manual_seed(5)
    T, IN, r, n = 300, 256, 16, 3
    segs = [128, 64, 64]
    x = _rand(T, IN)
    w = _rand(sum(segs), IN, scale=0.05)
    num_tokens = torch.tensor([100, 0, 200], dtype=torch.int32, device=DEV)

    def adapters(lead=()):
        out = []
        for i in range(n):
            a = (_rand(*lead, len(segs) * r, IN, scale=0.1)).requires_grad_()
            bl = [(_rand(*lead, s, r, scale=0.1)).requires_grad_() for s in segs]
            out.append((a, bl, 0.5 * (i + 1)))
        return out

    ad = adapters()
    xg = x.clone().requires_grad_()
    y = L.multi_lora_linear(xg, w, ad, num_tokens)
    dy = _rand(*y.shape)
    y.backward(dy)
    rt.check_status()
    ad_ref = [(a.detach().float().cpu().requires_grad_(), [b.detach().float().cpu().requires_grad_() for b in bl], sc)
              for a, bl, sc in ad]
    xr = x.float().cpu().requires_grad_()
    yr = L.multi_lora_linear(xr, w.float().cpu(), ad_ref, num_tokens.cpu())
    yr.backward(dy.float().cpu())
    _close(y.cpu(), yr, atol=0.05, rtol=2e-2)
    _close(xg.grad.cpu(), xr.grad, atol=0.05, rtol=3e-2)
    for (a, bl, _), (ar, blr, _) in zip(ad, ad_ref):            # bf16 intermediates (x A^T and its gradient)
        _close(a.grad.cpu(), ar.grad, atol=0.5, rtol=5e-2)
        assert float((a.grad.cpu().float() - ar.grad).norm() / (ar.grad.norm() + 1e-6)) < 0.03
        for b, br in zip(bl, blr):
            _close(b.grad.cpu(), br.grad, atol=0.5, rtol=5e-2)
    assert float(ad[1][0].grad.abs().sum()) == 0.0              # adapter 1 has no tokens

    # grouped: 3 experts, rows tagged with their adapter
    counts = torch.tensor([130, 5, 256], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    E = 3
    xp = _rand(P, IN)
    wg = _rand(E, sum(segs[:2]), IN, scale=0.05)
    segs2 = segs[:2]
    adg = []
    for i in range(2):
        a = _rand(E, len(segs2) * r, IN, scale=0.1).requires_grad_()
        bl = [_rand(E, s, r, scale=0.1).requires_grad_() for s in segs2]
        adg.append((a, bl, 1.0 + i))
    row_adapter = torch.randint(0, 2, (P,), device=DEV)
    row_adapter[::7] = -1
    yg = L.multi_lora_grouped_linear(xp, wg, adg, row_adapter, be.to(DEV), offs.to(DEV))
    dyg = _rand(*yg.shape)
    yg.backward(dyg)
    rt.check_status()
    adg_ref = [(a.detach().float().cpu().requires_grad_(), [b.detach().float().cpu().requires_grad_() for b in bl], sc)
               for a, bl, sc in adg]
    ygr = L.multi_lora_grouped_linear(xp.float().cpu(), wg.float().cpu(), adg_ref, row_adapter.cpu(), be, offs)
    ygr.backward(dyg.float().cpu())
    used = (be >= 0).repeat_interleave(128)
    _close(yg.cpu()[used], ygr[used], atol=0.05, rtol=2e-2)
    for (a, bl, _), (ar, blr, _) in zip(adg, adg_ref):
        _close(a.grad.cpu(), ar.grad, atol=0.5, rtol=5e-2)
        assert float((a.grad.cpu().float() - ar.grad).norm() / (ar.grad.norm() + 1e-6)) < 0.03
        for b, br in zip(bl, blr):
            _close(b.grad.cpu(), br.grad, atol=0.5, rtol=5e-2)


@pytest.mark.parametrize("window", [None, 100])
def test_flash_attention_with_sinks_matches_reference(window):
    """A per-head sink logit joins the softmax denominator in the kernel's epilogue; outputs and every gradient
    (q, k, v and the sinks themselves) against the fp32 definition."""
    from prime_rl_b200.ops import attention as A

    torch.manual_seed(2)
    lens = [200, 333, 57]
    T, Hq, Hkv, D = sum(lens), 8, 2, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _rand(T, Hq, D).requires_grad_(), _rand(T, Hkv, D).requires_grad_(), _rand(T, Hkv, D).requires_grad_()
    sinks = (torch.randn(Hq, device=DEV) * 2).to(torch.bfloat16).requires_grad_()
    out = A.attention(q, k, v, cu, max(lens), window=window, sinks=sinks, backend="tcgen05")
    do = _rand(T, Hq, D)
    out.backward(do)
    rt.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sr = sinks.detach().float().requires_grad_()
    ref = A.attention_ref(qr, kr, vr, cu, window=window, sinks=sr)
    ref.backward(do.float())
    _close(out, ref, atol=2e-2, rtol=2e-2)
    _close(q.grad, qr.grad, atol=3e-2, rtol=3e-2)
    _close(k.grad, kr.grad, atol=6e-2, rtol=3e-2)
    _close(v.grad, vr.grad, atol=6e-2, rtol=3e-2)
    _close(sinks.grad, sr.grad, atol=0.15, rtol=5e-2)


def test_newton_schulz_on_the_tcgen05_gemm_matches_the_matmul_form():
    from prime_rl_b200.trainer.optim import newton_schulz

    torch.manual_seed(0)
    for shape in ((256, 512), (768, 256)):
        g = torch.randn(*shape, device=DEV)
        got = newton_schulz(g)
        rt.check_status()
        ref = newton_schulz(g.cpu()).to(DEV)                 # fp32 matmul form
        assert got.shape == g.shape
        assert float((got - ref).norm() / ref.norm()) < 0.05  # bf16 iterations against fp32
        s = torch.linalg.svdvals(got.float())
        assert float(s.max()) < 1.3 and float(s.min()) > 0.3  # roughly orthogonal, as the quintic leaves it


def test_weight_gradient_accumulation_through_tma_reduce_adds():
    """fp32 accumulators take the weight-gradient tiles as TMA reduce-adds (no read-back of C): widths that end
    inside a 32-column chunk, repeated accumulation, alpha, experts without rows, and an accumulator that is a
    strided view of a larger buffer."""
    from prime_rl_b200.ops import lora as L
    from prime_rl_b200.ops import matmul as mm

    torch.manual_seed(4)
    # dense: C[M, N] += alpha * A^T B, A [T, M], B [T, N]
    for T, M, N in ((333, 256, 520), (1024, 384, 2048), (90, 128, 36)):
        a, b = _rand(T, M), _rand(T, N)
        big = torch.randn(M, N + 12, device=DEV)
        acc = big[:, 4:4 + N]                                   # row pitch N + 12 (multiple of 4), 16-byte aligned start
        ref = acc.clone()
        for _ in range(3):
            mm.gemm(a, b, a_mn=True, b_mn=True, out=acc, alpha=0.5, beta=1.0)
            ref = ref + 0.5 * (a.float().t() @ b.float())
        rt.check_status()
        _close(acc, ref, atol=0.02 * T ** 0.5, rtol=1e-2)
        assert torch.equal(big[:, :4], big[:, :4]) and bool(torch.isfinite(big).all())
    # k-grouped: out[e] += dy_e^T x_e, rows per expert a multiple of 128 so that tiles never straddle experts
    counts = torch.tensor([130, 0, 5, 256, 700], dtype=torch.int32)
    offs, be, P = _blocks(counts)
    E, M, N = 5, 256, 200
    valid = (be >= 0).repeat_interleave(128).to(DEV)
    dy = _rand(P, M) * valid[:, None]
    x = _rand(P, N) * valid[:, None]
    acc = torch.full((E, M, N), 2.0, device=DEV)
    ref = acc.clone()
    o = offs.tolist()
    for _ in range(2):
        L.kgrouped_gemm(dy, x, offs.to(DEV), E, out=acc, beta=1.0)
        for e in range(E):
            ref[e] += dy[o[e]:o[e + 1]].float().t() @ x[o[e]:o[e + 1]].float()
    rt.check_status()
    _close(acc, ref, atol=0.5, rtol=1e-2)
    assert torch.equal(acc[1], torch.full((M, N), 2.0, device=DEV))


@pytest.mark.gpu
def test_fp8_training_linear_and_grouped_linear_on_the_fp8_kernel():
    """Forward product and input gradient through the block-scaled fp8 kernel stay within e4m3 accuracy of the bf16
    products; the weight gradient (bf16 product into the fp32 accumulator) is the exact one."""
    from prime_rl_b200.ops import fp8 as F
    from prime_rl_b200 import ops

    torch.manual_seed(3)
    F.bump_weight_epoch()
    x = _rand(1000, 2048).requires_grad_()
    w = (_rand(1536, 2048) * 0.05).requires_grad_()
    dy = _rand(1000, 1536)
    y = F.fp8_linear(x, w)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    ref = x.float() @ w.float().t()
    rx, rw = torch.autograd.grad(ref, (x, w), dy.float())
    rt.check_status()
    for got, want, tol in ((y, ref, 0.06), (gx, rx, 0.06), (gw, rw, 0.01)):
        rel = float((got.float() - want.float()).norm() / want.float().norm())
        assert rel < tol, rel

    E, N, K = 4, 768, 2048
    block_expert = torch.tensor([0, 0, 1, 3, 3, 3, -1], dtype=torch.int32, device=DEV)
    expert_offset = torch.tensor([0, 256, 384, 384, 768], dtype=torch.int32, device=DEV)
    xp = _rand(7 * 128, K).requires_grad_()
    we = (_rand(E, N, K) * 0.05).requires_grad_()
    dyp = _rand(7 * 128, N)
    dyp[768:] = 0
    yp = F.fp8_grouped_linear(xp, we, block_expert, expert_offset)
    gxp, gwe = torch.autograd.grad(yp, (xp, we), dyp)
    yr = ops.grouped_linear(xp, we, block_expert, expert_offset)
    rxp, rwe = torch.autograd.grad(yr, (xp, we), dyp)
    rt.check_status()
    for got, want, tol in ((yp[:768], yr[:768], 0.06), (gxp[:768], rxp[:768], 0.06), (gwe, rwe, 0.01)):
        rel = float((got.float() - want.float()).norm() / want.float().norm())
        assert rel < tol, rel



@pytest.mark.gpu
@pytest.mark.parametrize("deterministic", [False, True])
def test_moe_plan_over_an_expert_range_sums_to_the_full_plan(deterministic):
    """Serving-side expert parallelism: plans over disjoint expert ranges (pairs of other experts get slot -1 and no
    row) give partial outputs that add up to the output of the plan over all experts."""
    T, k, E, H = 300, 4, 16, 256
    torch.manual_seed(5)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    w = torch.rand(T, k, device=DEV)
    x = _rand(T, H)
    full = moe.build_plan(idx, counts, E, deterministic=deterministic)
    y_full = moe.combine(moe.permute(x, full) * 2.0, w, full, T).float()
    total = torch.zeros_like(y_full)
    for lo, hi in ((0, 4), (4, 5), (5, 16)):
        plan = moe.build_plan(idx, counts, E, deterministic=deterministic, expert_range=(lo, hi))
        own = (idx >= lo) & (idx < hi)
        assert torch.equal(plan.slot >= 0, own)
        assert int(plan.total_rows) == int(((counts[lo:hi] + 127) // 128 * 128).sum())
        src = plan.row_src[plan.row_src >= 0].long()
        assert src.numel() == int(own.sum()) and bool(own.reshape(-1)[src].all())
        be = plan.block_expert[plan.block_expert >= 0]
        assert int(be.max()) < hi - lo
        total += moe.combine(moe.permute(x, plan) * 2.0, w, plan, T).float()
    rt.check_status()
    _close(total, y_full, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_recurrence_step_kernels_match_the_pytorch_steps():
    """Decode-step kernels of the state-carrying mixers (in place on pooled states, sequences addressed by slot)."""
    from prime_rl_b200.ops import delta_rule, ssm

    torch.manual_seed(9)
    lib = rt.lib()
    n, H, P, N, G, cap = 5, 8, 64, 128, 2, 11
    slots = torch.tensor([7, 0, 3, 10, 4], dtype=torch.int32, device=DEV)
    pool = torch.randn(cap, H, P, N, device=DEV)
    x, dt = torch.randn(n, H, P, device=DEV), torch.rand(n, H, device=DEV) * 0.1
    A, D = -torch.rand(H, device=DEV), torch.randn(H, device=DEV)
    B, C = torch.randn(n, G, N, device=DEV), torch.randn(n, G, N, device=DEV)
    want_y, want_s = ssm.mamba2_step(x, dt, A, B, C, D, pool[slots.long()])
    before = pool.clone()
    y = torch.empty(n, H, P, device=DEV)
    rt.check(lib.prb_mamba2_step(pool.data_ptr(), slots.data_ptr(), x.data_ptr(), dt.data_ptr(), A.data_ptr(),
                                 B.data_ptr(), C.data_ptr(), D.data_ptr(), y.data_ptr(), n, H, P, N, G,
                                 rt.stream_ptr(torch.device(DEV))), "prb_mamba2_step")
    _close(y, want_y, atol=1e-3, rtol=1e-3)
    _close(pool[slots.long()], want_s, atol=1e-4, rtol=1e-4)
    untouched = [i for i in range(cap) if i not in slots.tolist()]
    assert torch.equal(pool[untouched], before[untouched])

    dk, dv = 128, 96
    pool = torch.randn(cap, H, dk, dv, device=DEV) * 0.1
    q, k, v = torch.randn(n, H, dk, device=DEV), torch.randn(n, H, dk, device=DEV), torch.randn(n, H, dv, device=DEV)
    g, beta = -torch.rand(n, H, device=DEV), torch.rand(n, H, device=DEV)
    want_o, want_s = delta_rule.gated_delta_rule_step(q, k, v, g, beta, pool[slots.long()])
    qf = (delta_rule._l2norm(q) * dk ** -0.5).contiguous()
    kf = delta_rule._l2norm(k).contiguous()
    o = torch.empty(n, H, dv, device=DEV)
    rt.check(lib.prb_delta_rule_step(pool.data_ptr(), slots.data_ptr(), qf.data_ptr(), kf.data_ptr(), v.data_ptr(),
                                     g.data_ptr(), beta.data_ptr(), o.data_ptr(), n, H, dk, dv,
                                     rt.stream_ptr(torch.device(DEV))), "prb_delta_rule_step")
    _close(o, want_o, atol=1e-4, rtol=1e-3)
    _close(pool[slots.long()], want_s, atol=1e-4, rtol=1e-3)
