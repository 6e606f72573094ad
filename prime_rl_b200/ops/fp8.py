"""Block-scaled fp8 (e4m3) linear algebra: 1 x 128 activation scales, 128 x 128 weight scales
(``csrc/gemm_fp8.cu``; weights are quantised with ``models/fp8.py`` or in flight by the weight
push). Inference only: there is no backward."""

from __future__ import annotations

import torch

from . import _runtime as rt


def quantize_act(x: torch.Tensor, row_valid: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """x bf16 [M, K] -> (e4m3 as uint8 [M, K], fp32 scales [M, ceil(K/128)]). ``row_valid`` (int32 [M]):
    rows with a negative entry are padding; on a GPU they are neither read nor written."""
    M, K = x.shape
    KB = (K + 127) // 128
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x if x.stride(1) == 1 else x.contiguous()
        q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
        s = torch.empty(M, KB, dtype=torch.float32, device=x.device)
        rt.check(rt.lib().prb_act_quant_fp8(x.data_ptr(), x.stride(0), q.data_ptr(), s.data_ptr(), M, K,
                                            rt.ptr(row_valid), rt.stream_ptr(x.device)), "prb_act_quant_fp8")
        return q, s
    pad = torch.zeros(M, KB * 128, dtype=torch.float32, device=x.device)
    pad[:, :K] = x.float() if row_valid is None else torch.where((row_valid >= 0)[:, None], x.float(), 0.0)
    blocks = pad.view(M, KB, 128)
    s = blocks.abs().amax(-1).clamp_min(1e-12) / 448.0
    q = (blocks / s[..., None]).view(M, KB * 128)[:, :K].to(torch.float8_e4m3fn)
    return q.view(torch.uint8), s


def fp8_gemm_ref(aq, sa, bq, sb, block_expert=None) -> torch.Tensor:
    """fp32 reference: dequantise, then multiply. bq: [N, K] or [E, N, K] (uint8 / float8)."""
    a = aq.view(torch.float8_e4m3fn).float() * sa.repeat_interleave(128, 1)[:, :aq.shape[1]]

    def deq(bq_e, sb_e):
        N, K = bq_e.shape
        s = sb_e.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
        return bq_e.view(torch.float8_e4m3fn).float() * s

    if block_expert is None:
        return a @ deq(bq, sb).t()
    out = torch.zeros(a.shape[0], bq.shape[1], dtype=torch.float32, device=a.device)
    for blk, e in enumerate(block_expert.tolist()):
        if e >= 0:
            rows = slice(blk * 128, min((blk + 1) * 128, a.shape[0]))
            out[rows] = a[rows] @ deq(bq[e], sb[e]).t()
    return out


def fp8_gemm(aq, sa, bq, sb, *, block_expert: torch.Tensor | None = None, out: torch.Tensor | None = None,
             row_valid: torch.Tensor | None = None) -> torch.Tensor:
    """C bf16 [M, N] = dequant(aq, sa) @ dequant(bq, sb)^T. Grouped when ``block_expert`` is given
    (``bq`` [E, N, K], ``sb`` [E, ceil(N/128), ceil(K/128)], rows in 128-row expert blocks).
    ``row_valid`` (int32 [M]): rows with a negative entry are padding whose inputs may be uninitialised
    and whose outputs are not stored."""
    M, K = aq.shape
    N = bq.shape[-2]
    if not aq.is_cuda:
        if row_valid is not None:           # padding rows may hold anything: keep them out of the arithmetic
            aq, sa = aq.clone(), sa.clone()
            aq[row_valid < 0] = 0
            sa[row_valid < 0] = 0
        return fp8_gemm_ref(aq, sa, bq, sb, block_expert).to(torch.bfloat16)
    assert aq.is_contiguous() and bq.is_contiguous() and sa.is_contiguous() and sb.is_contiguous()
    assert bq.shape[-1] == K and K % 16 == 0
    E = bq.shape[0] if block_expert is not None else 1
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    status = rt.status_tensor(aq.device)
    rt.check(rt.lib().prb_gemm_fp8(aq.data_ptr(), sa.data_ptr(), bq.data_ptr(), sb.data_ptr(), out.data_ptr(), M, N, K,
                                   out.stride(0), rt.ptr(block_expert), E, rt.ptr(row_valid), status.data_ptr(),
                                   rt.stream_ptr(aq.device)),
             "prb_gemm_fp8")
    return out
