"""Fused LM head: per-token log-probability of the label and entropy of the (temperature
scaled) next-token distribution, without materialising the logits in the forward pass.

GPU path (``csrc/gemm.cu``): the ``h @ W^T`` tiles stay in tensor memory; the epilogue keeps
per-row running (max, sum exp, sum exp*z) over vocabulary splits; a small kernel merges the
splits. Backward rebuilds the logits tile by tile and writes
``dlogits = g * inv_temp * (onehot - softmax)`` in bf16, then two GEMMs give ``dh`` and ``dW``.
Entropy carries no gradient, as in the reference
(src/prime_rl/trainer/models/layers/lm_head.py:114-266).
"""

from __future__ import annotations

import torch

from . import _runtime as rt
from .matmul import gemm, grad_accumulator


def logprob_entropy_ref(h, w, labels, inv_temp=None, chunk: int = 4096):
    """fp32 reference; chunks tokens so that CPU tests on larger shapes stay small."""
    T = h.shape[0]
    lps, ents = [], []
    for s in range(0, T, chunk):
        z = h[s:s + chunk].float() @ w.float().t()
        if inv_temp is not None:
            z = z * inv_temp[s:s + chunk].float()[:, None]
        lse = torch.logsumexp(z, dim=-1)
        lb = labels[s:s + chunk].long()
        valid = (lb >= 0) & (lb < w.shape[0])
        tgt = z.gather(1, lb.clamp(0, w.shape[0] - 1)[:, None]).squeeze(1)
        lps.append(torch.where(valid, tgt - lse, torch.zeros_like(lse)))
        p = torch.softmax(z, dim=-1)
        ents.append(lse - (p * z).sum(-1))
    return torch.cat(lps), torch.cat(ents).detach()


class _FusedLogprobEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, inv_temp):
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        splits = rt.lib().prb_lmhead_num_splits(T, V)
        part = torch.empty(3, splits, T, dtype=torch.float32, device=dev)
        target = torch.empty(T, dtype=torch.float32, device=dev)
        out = torch.empty(3, T, dtype=torch.float32, device=dev)
        status = rt.status_tensor(dev)
        rc = rt.lib().prb_lmhead_fwd(h.data_ptr(), w.data_ptr(), labels.data_ptr(), rt.ptr(inv_temp),
                                     part[0].data_ptr(), part[1].data_ptr(), part[2].data_ptr(), target.data_ptr(),
                                     out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), T, V, H,
                                     h.stride(0), w.stride(0), splits, status.data_ptr(), rt.stream_ptr(dev))
        rt.check(rc, "prb_lmhead_fwd")
        ctx.save_for_backward(h, w, labels, inv_temp, out[2])
        ctx.grad_acc = grad_accumulator(w) if w.requires_grad else None
        ctx.mark_non_differentiable(out[1])
        return out[0], out[1]

    @staticmethod
    def backward(ctx, g_lp, _g_ent):
        h, w, labels, inv_temp, lse = ctx.saved_tensors
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        Vp = (V + 7) // 8 * 8
        dlogits = torch.empty(T, Vp, dtype=torch.bfloat16, device=dev)
        if Vp != V:
            dlogits[:, V:].zero_()
        g = g_lp.contiguous().float()
        status = rt.status_tensor(dev)
        rc = rt.lib().prb_lmhead_bwd_dlogits(h.data_ptr(), w.data_ptr(), labels.data_ptr(), rt.ptr(inv_temp),
                                             g.data_ptr(), lse.data_ptr(), dlogits.data_ptr(), T, V, H, h.stride(0),
                                             w.stride(0), dlogits.stride(0), status.data_ptr(), rt.stream_ptr(dev))
        rt.check(rc, "prb_lmhead_bwd_dlogits")
        dl = dlogits[:, :V]
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh = gemm(dl, w, b_mn=True)
        if ctx.needs_input_grad[1]:
            if ctx.grad_acc is not None and H % 4 == 0:
                gemm(dl, h, a_mn=True, b_mn=True, out=ctx.grad_acc, beta=1.0)      # added in place, no bf16 dW
            else:
                dw = gemm(dl, h, a_mn=True, b_mn=True)
        return dh, dw, None, None


def fused_logprob_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                          inv_temp: torch.Tensor | None = None):
    """h: [T, H]; w: [V, H]; labels: [T] (ids outside [0, V) give logprob 0); inv_temp: [T].
    Returns fp32 ``(logprob [T], entropy [T])``; only ``logprob`` is differentiable."""
    if h.is_cuda and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        h = h.contiguous()
        lab = labels.to(torch.int32).contiguous()
        it = inv_temp.float().contiguous() if inv_temp is not None else None
        return _FusedLogprobEntropy.apply(h, w, lab, it)
    return logprob_entropy_ref(h, w, labels, inv_temp)


def sampling_replay_rows(sampling_mask: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Rows whose sampling mask can be replayed: not empty (-1 = padding) and containing the label
    (a label outside its mask means misaligned data; such rows keep the full-vocabulary value)."""
    return (sampling_mask >= 0).any(-1) & (sampling_mask == labels.unsqueeze(-1)).any(-1)


def replay_sampling_mask(logprobs: torch.Tensor, h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                         inv_temp: torch.Tensor | None, sampling_mask: torch.Tensor,
                         bytes_budget: int = 1 << 29) -> torch.Tensor:
    """Renormalises ``logprobs [T]`` over the ids the rollout engine actually sampled from
    (``sampling_mask [T, K]`` int, -1 padded; top-k / top-p / min-p truncation): replayable rows get
    ``z[label] - logsumexp(z[mask ids])``, the rest keep their full-vocabulary value. Only the
    ``K`` masked logits per row are recomputed (rows of ``w`` gathered in blocks of tokens), so the
    fused head stays fused. Same contract as the reference's mask replay
    (src/prime_rl/trainer/models/layers/lm_head.py:97-111, :167-198; trainer/rl/loss.py:66-84)."""
    T, K = sampling_mask.shape
    H = h.shape[1]
    lab = labels.long()
    replay = sampling_replay_rows(sampling_mask, lab)
    ids = sampling_mask.clamp_min(0).long()
    block = max(1, bytes_budget // max(1, K * H * w.element_size()))
    outs = []
    for t0 in range(0, T, block):
        t1 = min(T, t0 + block)
        hb = h[t0:t1]
        z = torch.einsum("th,tkh->tk", hb.float(), w[ids[t0:t1]].float())
        tgt = (hb.float() * w[lab[t0:t1].clamp(0, w.shape[0] - 1)].float()).sum(-1)
        if inv_temp is not None:
            it = inv_temp[t0:t1].float()
            z, tgt = z * it[:, None], tgt * it
        z = torch.where(sampling_mask[t0:t1] >= 0, z, torch.full_like(z, float("-inf")))
        z = torch.where(replay[t0:t1, None], z, torch.zeros_like(z))     # keeps the unused branch finite
        outs.append(tgt - torch.logsumexp(z, dim=-1))
    return torch.where(replay, torch.cat(outs), logprobs)


def softcapped_logprob_entropy(h, w, labels, inv_temp=None, softcap: float = 30.0, chunk: int = 2048):
    """Head with ``softcap * tanh(z / softcap)`` applied to the logits before temperature scaling
    (Gemma family; src/prime_rl/trainer/models/layers/lm_head_gemma.py). Token-chunked, with the
    chunk's logits recomputed in backward by checkpointing, so at most ``chunk x V`` logits exist."""
    from torch.utils.checkpoint import checkpoint

    def piece(hc, lc, ic):
        z = softcap * torch.tanh((hc.float() @ w.float().t()) / softcap)
        if ic is not None:
            z = z * ic.float()[:, None]
        lse = torch.logsumexp(z, dim=-1)
        lb = lc.long()
        valid = (lb >= 0) & (lb < w.shape[0])
        tgt = z.gather(1, lb.clamp(0, w.shape[0] - 1)[:, None]).squeeze(1)
        lp = torch.where(valid, tgt - lse, torch.zeros_like(lse))
        with torch.no_grad():
            ent = lse - (torch.softmax(z, dim=-1) * z).sum(-1)
        return lp, ent

    lps, ents = [], []
    for s in range(0, h.shape[0], chunk):
        ic = inv_temp[s:s + chunk] if inv_temp is not None else None
        if torch.is_grad_enabled() and (h.requires_grad or w.requires_grad):
            lp, ent = checkpoint(piece, h[s:s + chunk], labels[s:s + chunk], ic, use_reentrant=False)
        else:
            lp, ent = piece(h[s:s + chunk], labels[s:s + chunk], ic)
        lps.append(lp)
        ents.append(ent.detach())
    return torch.cat(lps), torch.cat(ents)
