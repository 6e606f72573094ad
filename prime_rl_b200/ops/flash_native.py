"""Front end of the hand-written flash-attention kernels (``csrc/flash_attn.cu``)."""

from __future__ import annotations

import math

import torch

from .. import native
from . import _runtime as rt


def available() -> bool:
    try:
        return hasattr(native.cuda(), "prb_flash_fwd")
    except Exception:
        return False


def flash_fwd(q, k, v, cu_seqlens, *, scale: float | None = None, window: int | None = None,
              q_offset: int | None = None, sinks: torch.Tensor | None = None):
    """q: [T, Hq, 128] bf16 (contiguous heads), k/v: [T, Hkv, 128] bf16 (may be strided over
    tokens). Returns (out [T, Hq, 128] bf16, lse [Hq, T] fp32, natural log).

    Context-parallel form (``q_offset`` given): ``q`` holds only the global rows
    ``[q_offset, q_offset + q.shape[0])`` while k / v / cu_seqlens describe the whole sequence;
    out and lse are for the held rows. ``sinks`` (fp32 [Hq]): a per-head logit that joins every row's softmax
    denominator (and therefore ``lse``) without a value."""
    Tq, Hq, D = q.shape
    T = k.shape[0]
    Hkv = k.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == D, "heads must be contiguous"
    off = 0 if q_offset is None else int(q_offset)
    assert q_offset is not None or Tq == T
    out = torch.empty(Tq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    num_docs = cu_seqlens.numel() - 1
    max_pairs = (T + 255) // 256 + num_docs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == Hq and sinks.is_contiguous()
    status = rt.status_tensor(q.device)
    rc = rt.lib().prb_flash_fwd_slice(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      cu_seqlens.data_ptr(), num_docs, T, off, Tq, Hq, Hkv, D, q.stride(0),
                                      k.stride(0), v.stride(0), out.stride(0), float(scale), int(window or 0),
                                      max_pairs, rt.ptr(sinks), status.data_ptr(), rt.stream_ptr(q.device))
    rt.check(rc, "prb_flash_fwd_slice")
    return out, lse


def flash_fwd_block(q, k, v, cu_seqlens, total: int, q_offset: int, k_offset: int, *, scale: float | None = None,
                    window: int | None = None):
    """Partial attention of the global rows ``[q_offset, q_offset + Tq)`` over the keys ``[k_offset, k_offset + Tk)``
    of a packed sequence of ``total`` tokens (``cu_seqlens`` describes the whole sequence; causal and document masks
    by global position). Returns (out [Tq, Hq, 128] bf16, lse [Hq, Tq] fp32): rows that see none of the keys come
    back as out = 0, lse = -inf. One step of the ring form of context parallelism (``merge_partial`` combines)."""
    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == D, "heads must be contiguous"
    out = torch.empty(Tq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    num_docs = cu_seqlens.numel() - 1
    max_pairs = (total + 255) // 256 + num_docs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    status = rt.status_tensor(q.device)
    rc = rt.lib().prb_flash_fwd_block(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      cu_seqlens.data_ptr(), num_docs, int(total), int(q_offset), Tq, int(k_offset), Tk,
                                      Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), out.stride(0), float(scale),
                                      int(window or 0), max_pairs, None, status.data_ptr(), rt.stream_ptr(q.device))
    rt.check(rc, "prb_flash_fwd_block")
    return out, lse


def flash_bwd_block(dout, q, k, v, out, lse, cu_seqlens, total: int, q_offset: int, k_offset: int, *,
                    scale: float | None = None, window: int | None = None):
    """Partial gradients of one (row slice, key range) block: ``out`` / ``lse`` are the rows' FINAL output and
    log-sum-exp over all keys. Returns (dq [Tq, Hq, 128], dk, dv [Tk, Hkv, 128]) in bf16; the caller sums the blocks."""
    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16
    dout = dout.contiguous()
    for t in (q, k, v, out, dout):
        assert t.stride(2) == 1 and t.stride(1) == D, "heads must be contiguous"
    dev = q.device
    dq = torch.empty(Tq, Hq, D, dtype=q.dtype, device=dev)
    dk = torch.zeros(Tk, Hkv, D, dtype=q.dtype, device=dev)
    dv = torch.zeros(Tk, Hkv, D, dtype=q.dtype, device=dev)
    delta = torch.empty(Hq, Tq, dtype=torch.float32, device=dev)
    num_docs = cu_seqlens.numel() - 1
    max_blocks = (total + 127) // 128 + num_docs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    status = rt.status_tensor(dev)
    rc = rt.lib().prb_flash_bwd_block(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                      lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                      cu_seqlens.data_ptr(), num_docs, int(total), int(q_offset), Tq, int(k_offset), Tk,
                                      Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), out.stride(0), dout.stride(0),
                                      dk.stride(0), dv.stride(0), float(scale), int(window or 0), max_blocks,
                                      status.data_ptr(), rt.stream_ptr(dev))
    rt.check(rc, "prb_flash_bwd_block")
    return dq, dk, dv


def flash_fwd_gather(q, k_full, v_full, peer_ptrs, cu_seqlens, cp_rank: int, cp_size: int, counters, *,
                     scale: float | None = None, window: int | None = None):
    """Context-parallel forward with the K / V exchange inside the kernel. ``k_full`` / ``v_full``
    ``[T, Hkv, 128]`` are the two halves of ONE buffer per rank (``v_full`` directly after ``k_full``
    or at any 16-byte aligned distance) in which this rank has written the rows of its own chunk;
    ``peer_ptrs`` is a ctypes array with the address of that buffer (its ``k_full``) on every rank.
    ``q [T / cp, Hq, 128]`` are the local rows. After the call the chunks of all lower ranks are
    present in the local buffer as well. Returns (out, lse) for the local rows."""
    Tq, Hq, D = q.shape
    T, Hkv = k_full.shape[0], k_full.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16 and T == Tq * cp_size
    assert k_full.is_contiguous() and v_full.is_contiguous() and q.stride(2) == 1 and q.stride(1) == D
    v_off = v_full.data_ptr() - k_full.data_ptr()
    out = torch.empty(Tq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    num_docs = cu_seqlens.numel() - 1
    max_pairs = (T + 255) // 256 + num_docs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    status = rt.status_tensor(q.device)
    rc = rt.lib().prb_flash_fwd_gather(q.data_ptr(), k_full.data_ptr(), peer_ptrs, v_off, out.data_ptr(), lse.data_ptr(),
                                       cu_seqlens.data_ptr(), num_docs, T, Hq, Hkv, q.stride(0), out.stride(0),
                                       float(scale), int(window or 0), max_pairs, cp_rank, cp_size, Tq,
                                       counters.data_ptr(), status.data_ptr(), rt.stream_ptr(q.device))
    rt.check(rc, "prb_flash_fwd_gather")
    return out, lse


def bwd_available() -> bool:
    try:
        return hasattr(native.cuda(), "prb_flash_bwd")
    except Exception:
        return False


def flash_bwd(dout, q, k, v, out, lse, cu_seqlens, *, scale: float | None = None, window: int | None = None,
              dk_out: torch.Tensor | None = None, dv_out: torch.Tensor | None = None, q_offset: int | None = None):
    """Returns (dq [Tq, Hq, 128], dk, dv [T, Hkv, 128]) in bf16. With ``q_offset`` the query-side
    tensors hold the global rows ``[q_offset, q_offset + Tq)`` only and dk / dv are this
    rank's contributions for all T keys."""
    Tq, Hq, D = q.shape
    T = k.shape[0]
    Hkv = k.shape[1]
    assert D == 128 and q.dtype == torch.bfloat16
    dout = dout.contiguous()
    for t in (q, k, v, out, dout):
        assert t.stride(2) == 1 and t.stride(1) == D, "heads must be contiguous"
    off = 0 if q_offset is None else int(q_offset)
    dev = q.device
    dq = torch.empty(Tq, Hq, D, dtype=q.dtype, device=dev)
    dk = dk_out if dk_out is not None else torch.empty(T, Hkv, D, dtype=q.dtype, device=dev)
    dv = dv_out if dv_out is not None else torch.empty(T, Hkv, D, dtype=q.dtype, device=dev)
    delta = torch.empty(Hq, Tq, dtype=torch.float32, device=dev)
    num_docs = cu_seqlens.numel() - 1
    max_blocks = (T + 127) // 128 + num_docs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    status = rt.status_tensor(dev)
    rc = rt.lib().prb_flash_bwd_slice(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                      lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                      cu_seqlens.data_ptr(), num_docs, T, off, Tq, Hq, Hkv, D, q.stride(0),
                                      k.stride(0), v.stride(0), out.stride(0), dout.stride(0), dk.stride(0),
                                      dv.stride(0), float(scale), int(window or 0), max_blocks, status.data_ptr(),
                                      rt.stream_ptr(dev))
    rt.check(rc, "prb_flash_bwd_slice")
    return dq, dk, dv
