"""Block-scaled fp8 (e4m3) weights: 128 x 128 blocks, one fp32 scale per block,
``scale = amax / 448`` and ``weight ~ q * scale`` — the layout of DeepSeek-style fp8
checkpoints (``<name>`` in float8_e4m3fn plus ``<name>_scale_inv`` in fp32; reference:
src/prime_rl/trainer/models/fp8.py:1-64).

On a GPU the quantiser is the same kernel the peer-memory weight push uses
(``csrc/weight_push.cu``), pointed at local memory."""

from __future__ import annotations

import torch

BLOCK = 128
FP8_MAX = 448.0


def quantize_to_fp8_blockwise(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w: [..., N, K] -> (q float8_e4m3fn same shape, scale_inv fp32 [..., ceil(N/128), ceil(K/128)])."""
    lead, (N, K) = w.shape[:-2], w.shape[-2:]
    w2 = w.reshape(-1, N, K)
    if w.is_cuda and w.dtype == torch.bfloat16 and K % 2 == 0:
        from ..ops import _runtime as rt

        q = torch.empty(w2.shape, dtype=torch.uint8, device=w.device)
        s = torch.empty(w2.shape[0], (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK, dtype=torch.float32,
                        device=w.device)
        for i in range(w2.shape[0]):
            wi = w2[i].contiguous()
            rt.check(rt.lib().prb_weight_push_fp8(wi.data_ptr(), wi.stride(0), q[i].data_ptr(), s[i].data_ptr(), N, K,
                                                  rt.stream_ptr(w.device)), "prb_weight_push_fp8")
        return q.view(torch.float8_e4m3fn).reshape(*lead, N, K), s.reshape(*lead, *s.shape[1:])
    pn, pk = (N + BLOCK - 1) // BLOCK * BLOCK, (K + BLOCK - 1) // BLOCK * BLOCK
    pad = torch.zeros(w2.shape[0], pn, pk, dtype=torch.float32, device=w.device)
    pad[:, :N, :K] = w2.float()
    blocks = pad.view(-1, pn // BLOCK, BLOCK, pk // BLOCK, BLOCK)
    scale = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-12) / FP8_MAX
    q = (blocks / scale[:, :, None, :, None]).view(-1, pn, pk)[:, :N, :K].to(torch.float8_e4m3fn)
    return q.reshape(*lead, N, K), scale.reshape(*lead, *scale.shape[1:])


def dequantize_fp8_blockwise(q: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    N, K = q.shape[-2:]
    s = scale_inv.repeat_interleave(BLOCK, -2)[..., :N, :].repeat_interleave(BLOCK, -1)[..., :K]
    return (q.float() * s).to(dtype)


def should_quantize(name: str, t: torch.Tensor) -> bool:
    """Linear / expert weights only: norms, embeddings, the LM head, routers and biases stay as they are."""
    if t.dim() < 2 or not name.endswith(("weight", "_proj")) and "proj" not in name:
        return False
    skip = ("embed_tokens", "lm_head", "norm", "router", "gate.weight", "e_score_correction")
    return not any(s in name for s in skip) and t.shape[-1] % 2 == 0


def quantize_state_dict(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    out = {}
    for name, t in sd.items():
        if should_quantize(name, t):
            q, s = quantize_to_fp8_blockwise(t.to(torch.bfloat16))
            out[name] = q
            out[name + "_scale_inv"] = s
        else:
            out[name] = t
    return out


def dequantize_state_dict(sd: dict[str, torch.Tensor], dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    out = {}
    for name, t in sd.items():
        if name.endswith("_scale_inv"):
            continue
        s = sd.get(name + "_scale_inv")
        out[name] = dequantize_fp8_blockwise(t, s, dtype) if s is not None else t
    return out
