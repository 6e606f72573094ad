"""Token sampling: per-request temperature, top-k / top-p truncation with capture of the kept
token ids (the "sampling mask" the trainer replays, <= 512 ids per position), and the
log-probability of the sampled token under the *processed* distribution — what the
reference asks of vLLM with ``logprobs_mode=processed_logprobs``
(packages/prime-rl-configs/src/prime_rl/configs/inference.py:602-654)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

MAX_MASK = 512


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_tokens: int = 0
    seed: int | None = None
    stop_token_ids: tuple[int, ...] = ()
    logprobs: int | None = 0
    prompt_logprobs: bool = False
    return_routed_experts: bool = False
    return_sampling_mask: bool = False

    @classmethod
    def from_dict(cls, d: dict | None) -> "SamplingParams":
        d = dict(d or {})
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        if "stop_token_ids" in known:
            known["stop_token_ids"] = tuple(known["stop_token_ids"])
        if "prompt_logprobs" in known:
            known["prompt_logprobs"] = bool(known["prompt_logprobs"])
        return cls(**known)

    @property
    def truncated(self) -> bool:
        return self.top_p < 1.0 or self.top_k > 0


def _draw_seed(generator: torch.Generator | None) -> int:
    """63-bit seed for the counter-based generator of the sampling kernel, drawn on the host: from the
    request's generator when it has one (so that a seeded request replays), else from the global CPU one."""
    if generator is not None and generator.device.type != "cpu":
        # advance the device generator's host-side state without launching anything
        offset = generator.get_offset()
        generator.set_offset(offset + 4)
        return (generator.initial_seed() ^ ((offset + 1) * 0x9E3779B97F4A7C15)) & ((1 << 63) - 1)
    return int(torch.empty((), dtype=torch.int64).random_(generator=generator)) & ((1 << 63) - 1)


def sample_untruncated(logits: torch.Tensor, temperature: torch.Tensor, generator: torch.Generator | None = None):
    """Temperature-only sampling in ONE kernel pass over fp32 logits [B, V] (Gumbel-max with a counter-based
    generator, online log-softmax for the sampled token's log-probability). Returns (tokens int64, logprobs)."""
    from ..ops import _runtime as rt

    B, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        logits = logits.float().contiguous()
    tok = torch.empty(B, dtype=torch.int32, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    rt.check(rt.lib().prb_sample_gumbel(logits.data_ptr(), temperature.data_ptr(), logits.stride(0), _draw_seed(generator),
                                        tok.data_ptr(), lp.data_ptr(), B, V, rt.stream_ptr(logits.device)),
             "prb_sample_gumbel")
    return tok.long(), lp


def sample_truncated(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                     generator: torch.Generator | None = None, want_mask: bool = False):
    """Top-k / top-p sampling on the GPU without a sort (``csrc/sampling.cu: sample_truncated_kernel``: radix
    descent to the smallest kept logit, then Gumbel-max over the kept tokens). The kept ids come back unordered."""
    from ..ops import _runtime as rt

    B, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        logits = logits.float().contiguous()
    dev = logits.device
    tok = torch.empty(B, dtype=torch.int32, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev)
    ids = cnt = None
    if want_mask:
        ids = torch.empty(B, MAX_MASK, dtype=torch.int32, device=dev)
        cnt = torch.zeros(B, dtype=torch.int32, device=dev)
    rt.check(rt.lib().prb_sample_truncated(
        logits.data_ptr(), temperature.float().contiguous().data_ptr(), top_k.to(torch.int32).contiguous().data_ptr(),
        top_p.float().contiguous().data_ptr(), logits.stride(0), _draw_seed(generator), tok.data_ptr(), lp.data_ptr(),
        rt.ptr(ids), rt.ptr(cnt), MAX_MASK, B, V, rt.stream_ptr(dev)), "prb_sample_truncated")
    mask_ids = None
    if want_mask:
        counts = cnt.clamp(max=MAX_MASK).tolist()
        mask_ids = [ids[b, :counts[b]] for b in range(B)]
    return tok.long(), lp, mask_ids


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           generator: torch.Generator | None = None, want_mask: bool = False, truncated: bool | None = None):
    """logits fp32 [B, V]; temperature/top_p fp32 [B]; top_k int [B] (<= 0 = off).
    Returns (tokens [B], logprobs [B], mask_ids list[Tensor] | None). Temperature 0 = greedy.
    ``truncated`` says whether any row uses top-k / top-p when the caller knows it on the host
    (saves a device round trip); None = look at the tensors."""
    B, V = logits.shape
    if truncated is None:
        truncated = bool(((top_k > 0) | (top_p < 1.0)).any())
    if not truncated and logits.is_cuda:
        tok, lp = sample_untruncated(logits, temperature.float().contiguous(), generator)
        return tok, lp, None
    if logits.is_cuda:
        return sample_truncated(logits, temperature, top_k, top_p, generator, want_mask)
    greedy = temperature <= 0
    t = torch.where(greedy, torch.ones_like(temperature), temperature)
    z = logits.float() / t[:, None]
    mask_ids = None
    if truncated:
        srt, idx = torch.sort(z, dim=-1, descending=True)
        probs = torch.softmax(srt, dim=-1)
        cum = probs.cumsum(-1)
        keep = (cum - probs) < top_p[:, None]                       # always keeps the first token
        k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V)).clamp(max=V)
        keep &= torch.arange(V, device=z.device)[None, :] < k[:, None]
        srt = srt.masked_fill(~keep, float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(1, idx, srt)
        if want_mask:
            counts = keep.sum(-1).clamp(max=MAX_MASK)
            mask_ids = [idx[b, : int(counts[b])].to(torch.int32) for b in range(B)]
    logp = torch.log_softmax(z, dim=-1)
    p = logp.exp()
    tok = torch.multinomial(p, 1, generator=generator).squeeze(1)
    tok = torch.where(greedy, z.argmax(-1), tok)
    return tok, logp.gather(1, tok[:, None]).squeeze(1), mask_ids
