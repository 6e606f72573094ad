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


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           generator: torch.Generator | None = None, want_mask: bool = False):
    """logits fp32 [B, V]; temperature/top_p fp32 [B]; top_k int [B] (<= 0 = off).
    Returns (tokens [B], logprobs [B], mask_ids list[Tensor] | None). Temperature 0 = greedy."""
    B, V = logits.shape
    greedy = temperature <= 0
    t = torch.where(greedy, torch.ones_like(temperature), temperature)
    z = logits.float() / t[:, None]
    truncated = bool(((top_k > 0) | (top_p < 1.0)).any())
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
