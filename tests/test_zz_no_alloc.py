"""The allocation-free LM-head entry point, called through its exported C symbol.

Some users of the native library cannot allocate device memory when they call it — a serving
worker that already gave all free GPU memory to its KV cache, or a host program that talks
to the shared object directly and has no tensor allocator. ``prb_lmhead_fwd_noalloc`` keeps
its scratch in a fixed array inside the library. This test runs it twice in a row (the
scratch is shared between calls and keeps old contents) and compares each result with the
regular entry point, which gets its scratch from the caller.
"""

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from prime_rl_b200 import native

    lib = ctypes.CDLL(str(native.CUDA_LIB))
    P, I, L = c_void_p, c_int, c_longlong
    lib.prb_lmhead_fwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, L, L, P, P]
    lib.prb_lmhead_fwd_noalloc.restype = c_int
    lib.prb_lmhead_fwd.argtypes = [P, P, P, P, P, P, P, P, P, P, P, I, I, I, L, L, I, P, P]
    lib.prb_lmhead_fwd.restype = c_int
    lib.prb_lmhead_num_splits.argtypes = [I, I]
    lib.prb_lmhead_num_splits.restype = c_int
    lib.prb_bind_device.argtypes = [I]
    lib.prb_bind_device.restype = c_int
    return lib


def _regular(lib, h, w, labels, inv_temp, status, stream):
    T, H = h.shape
    V = w.shape[0]
    splits = lib.prb_lmhead_num_splits(T, V)
    part = torch.empty(3, splits, T, dtype=torch.float32, device=h.device)
    target = torch.empty(T, dtype=torch.float32, device=h.device)
    out = torch.empty(3, T, dtype=torch.float32, device=h.device)
    rc = lib.prb_lmhead_fwd(h.data_ptr(), w.data_ptr(), labels.data_ptr(), inv_temp.data_ptr(), part[0].data_ptr(),
                            part[1].data_ptr(), part[2].data_ptr(), target.data_ptr(), out[0].data_ptr(),
                            out[1].data_ptr(), out[2].data_ptr(), T, V, H, h.stride(0), w.stride(0), splits,
                            status.data_ptr(), stream)
    assert rc == 0
    return out


def _noalloc(lib, h, w, labels, inv_temp, status, stream):
    T, H = h.shape
    out = torch.empty(3, T, dtype=torch.float32, device=h.device)   # outputs belong to the caller
    rc = lib.prb_lmhead_fwd_noalloc(h.data_ptr(), w.data_ptr(), labels.data_ptr(), inv_temp.data_ptr(),
                                    out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), T, w.shape[0], H,
                                    h.stride(0), w.stride(0), status.data_ptr(), stream)
    assert rc == 0
    return out


def test_noalloc_lm_head_matches_regular_entry_point_twice():
    lib = _load()
    dev = torch.device("cuda", 0)
    assert lib.prb_bind_device(0) == 0
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    # two different problems back to back: the second call must not see leftovers of the first
    for T, V, H in ((700, 5000, 512), (300, 32000, 256)):
        h = (torch.randn(T, H, device=dev, generator=g)).to(torch.bfloat16)
        w = (torch.randn(V, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        labels = torch.randint(0, V, (T,), device=dev, generator=g).to(torch.int32)
        labels[::5] = -100
        inv_temp = 0.5 + torch.rand(T, device=dev, generator=g)
        ref = _regular(lib, h, w, labels, inv_temp, status, stream)
        got = _noalloc(lib, h, w, labels, inv_temp, status, stream)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for a, b, name in zip(got, ref, ("logprob", "entropy", "lse")):
            err = (a - b).abs()
            assert bool((err <= 2e-2 + 1e-2 * b.abs()).all()), f"{name}: max err {err.max().item():.4g}"
        # and against an fp32 PyTorch computation of the same op
        z = (h.float() @ w.float().t()) * inv_temp[:, None]
        lse = torch.logsumexp(z, -1)
        assert bool(((got[2] - lse).abs() <= 2e-2 + 1e-2 * lse.abs()).all())


def test_noalloc_decode_shapes_after_a_call_that_dirtied_the_scratch():
    """Few rows and a large vocabulary ask for more vocabulary slices than the built-in scratch has;
    the entry point then re-spreads the tiles so that every slice it merges was written by this call.
    Runs after a larger call so that the shared array holds foreign values."""
    lib = _load()
    dev = torch.device("cuda", 0)
    assert lib.prb_bind_device(0) == 0
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(2)
    H, V = 256, 151936
    w = (torch.randn(V, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    for T in (2048, 256, 128, 512):         # the first call fills all 64 slices for 2048 rows
        h = (torch.randn(T, H, device=dev, generator=g) * 3.0).to(torch.bfloat16)
        labels = torch.randint(0, V, (T,), device=dev, generator=g).to(torch.int32)
        inv_temp = 0.5 + torch.rand(T, device=dev, generator=g)
        got = _noalloc(lib, h, w, labels, inv_temp, status, stream)
        ref = _regular(lib, h, w, labels, inv_temp, status, stream)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        z = (h.float() @ w.float().t()) * inv_temp[:, None]
        lse = torch.logsumexp(z, -1)
        lp = z.gather(1, labels.long()[:, None])[:, 0] - lse
        p = torch.softmax(z, -1)
        ent = lse - (p * z).sum(-1)
        for a, b, name in zip(got, (lp, ent, lse), ("logprob", "entropy", "lse")):
            err = (a - b).abs()
            assert bool((err <= 3e-2 + 1e-2 * b.abs()).all()), f"T={T} {name} vs fp32: max err {err.max().item():.4g}"
        for a, b, name in zip(got, ref, ("logprob", "entropy", "lse")):
            err = (a - b).abs()
            assert bool((err <= 2e-2 + 1e-2 * b.abs()).all()), f"T={T} {name} vs regular: max err {err.max().item():.4g}"


def test_noalloc_rejects_oversized_input():
    lib = _load()
    dev = torch.device("cuda", 0)
    lib.prb_bind_device(0)
    T = 8192 + 128
    h = torch.zeros(T, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=dev)
    labels = torch.zeros(T, dtype=torch.int32, device=dev)
    out = torch.zeros(3, T, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.prb_lmhead_fwd_noalloc(h.data_ptr(), w.data_ptr(), labels.data_ptr(), None, out[0].data_ptr(),
                                    out[1].data_ptr(), out[2].data_ptr(), T, 256, 64, 64, 64, status.data_ptr(),
                                    torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -20
