"""Per-token RL losses over packed micro-batches.

Every loss is a sum over tokens, so a packed micro-batch is processed in one vectorised
pass (no per-sequence loop and no host synchronisation); custom losses are the exception and
are called once per sequence, which is the contract the reference gives them
(src/prime_rl/trainer/rl/loss.py:140-423).

Components and normalisation: ``rl`` (policy gradient, chosen by ``trainer.loss``), ``ce``
(masked NLL) and ``ref_kl`` (reverse KL to a reference policy). Each component is divided by
its own *global* token count, which the trainer all-reduces before the micro-batch loop.
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch import Tensor


@dataclass
class LossInputs:
    trainer_logprobs: Tensor
    inference_logprobs: Tensor
    advantages: Tensor
    loss_mask: Tensor
    ref_logprobs: Tensor | None = None
    loss_weights: Tensor | None = None


@dataclass
class LossOutputs:
    loss: Tensor
    metrics: dict[str, Tensor] = field(default_factory=dict)


def shift_left(t: Tensor, pad_value: float = 0.0) -> Tensor:
    """labels[i] = ids[i + 1] along the last token dim (dim 0 for [T], dim 1 for [B, T, ...])."""
    dim = 0 if t.dim() == 1 else 1
    pad = torch.full_like(t.narrow(dim, 0, 1), pad_value)
    return torch.cat([t.narrow(dim, 1, t.shape[dim] - 1), pad], dim=dim)


def shift_right(t: Tensor, pad_value: float = 0.0) -> Tensor:
    dim = 0 if t.dim() == 1 else 1
    pad = torch.full_like(t.narrow(dim, 0, 1), pad_value)
    return torch.cat([pad, t.narrow(dim, 0, t.shape[dim] - 1)], dim=dim)


def _safe_mean(values: Tensor, mask: Tensor) -> Tensor:
    m = mask.to(values.dtype)
    return (values * m).sum() / m.sum().clamp_min(1.0)


def importance(trainer_logprobs: Tensor, inference_logprobs: Tensor):
    log_ratio = trainer_logprobs - inference_logprobs
    ratio = torch.exp(log_ratio)
    return log_ratio, ratio, ratio - log_ratio - 1


class IPOLoss:
    """Symmetric trust region on the probability difference, importance-ratio policy
    gradient, squared-log-ratio regulariser."""

    def __init__(self, config):
        self.config = config

    def loss(self, x: LossInputs) -> LossOutputs:
        c = self.config
        log_ratio, ratio, mismatch_kl = importance(x.trainer_logprobs, x.inference_logprobs)
        diff = (torch.exp(x.trainer_logprobs) - torch.exp(x.inference_logprobs)).abs()
        is_masked = diff.detach() > c.eps
        keep = x.loss_mask & ~is_masked
        pg = keep * (c.adv_tau * x.advantages) * ratio
        kl = x.loss_mask * log_ratio ** 2
        per_token = -pg + c.kl_tau * kl
        if x.loss_weights is not None:
            per_token = per_token * x.loss_weights
        return LossOutputs(per_token.sum(), {
            "masked_mismatch_kl": _safe_mean(mismatch_kl.detach(), x.loss_mask & is_masked),
            "unmasked_mismatch_kl": _safe_mean(mismatch_kl.detach(), keep),
            "is_masked": _safe_mean(is_masked.float(), x.loss_mask),
        })


class IcePopLoss:
    """Policy gradient inside a fixed importance-ratio acceptance band."""

    def __init__(self, config):
        self.config = config

    def loss(self, x: LossInputs) -> LossOutputs:
        c = self.config
        log_ratio, _, mismatch_kl = importance(x.trainer_logprobs, x.inference_logprobs)
        lo = torch.log(torch.tensor(c.ratio_low, device=log_ratio.device))
        hi = torch.log(torch.tensor(c.ratio_high, device=log_ratio.device))
        d = log_ratio.detach()
        is_masked = (d < lo) | (d > hi)
        keep = x.loss_mask & ~is_masked
        safe = torch.where(keep, log_ratio, torch.zeros_like(log_ratio))  # no 0 * inf
        per_token = -(keep * c.adv_tau * x.advantages * torch.exp(safe))
        if x.loss_weights is not None:
            per_token = per_token * x.loss_weights
        return LossOutputs(per_token.sum(), {
            "masked_mismatch_kl": _safe_mean(mismatch_kl.detach(), x.loss_mask & is_masked),
            "unmasked_mismatch_kl": _safe_mean(mismatch_kl.detach(), keep),
            "is_masked": _safe_mean(is_masked.float(), x.loss_mask),
        })


def ref_kl_loss_fn(x: LossInputs) -> LossOutputs:
    if x.ref_logprobs is None:
        raise ValueError("ref_kl loss requires ref_logprobs (use the 'opd' or 'opsd' algorithm)")
    log_ratio, ratio, mismatch_kl = importance(x.trainer_logprobs, x.inference_logprobs)
    diff = (torch.exp(x.trainer_logprobs) - torch.exp(x.inference_logprobs)).detach()
    is_masked = diff < -0.2
    drop = x.loss_mask & is_masked
    keep = x.loss_mask & ~is_masked
    ref_kl = x.ref_logprobs - x.trainer_logprobs
    per_token = -(keep * ref_kl.detach() * ratio) + 1e-3 * (x.loss_mask * log_ratio ** 2)
    if x.loss_weights is not None:
        per_token = per_token * x.loss_weights
    return LossOutputs(per_token.sum(), {
        "ref_kl/masked_mismatch_kl": _safe_mean(mismatch_kl.detach(), drop),
        "ref_kl/unmasked_mismatch_kl": _safe_mean(mismatch_kl.detach(), keep),
        "ref_kl/is_masked": _safe_mean(is_masked.float(), x.loss_mask),
        "ref_kl": _safe_mean(ref_kl.detach(), x.loss_mask),
    })


def ce_loss_fn(x: LossInputs) -> LossOutputs:
    nll = -x.trainer_logprobs
    weighted = nll if x.loss_weights is None else nll * x.loss_weights
    return LossOutputs((weighted * x.loss_mask).sum(), {"nll": _safe_mean(nll.detach(), x.loss_mask)})


def import_object(path: str) -> Any:
    mod, _, name = path.replace(":", ".").rpartition(".")
    return getattr(importlib.import_module(mod), name)


class CustomLoss:
    per_sequence = True

    def __init__(self, config):
        self.config = config
        self.fn: Callable = import_object(config.import_path)

    def loss(self, x: LossInputs) -> LossOutputs:
        return self.fn(x, **self.config.kwargs)


def setup_rl_loss_fn(config):
    t = getattr(config, "type", None)
    if t == "ipo":
        return IPOLoss(config)
    if t == "icepop":
        return IcePopLoss(config)
    if t == "custom":
        return CustomLoss(config)
    raise TypeError(f"unsupported RL loss config: {type(config).__name__}")


def compute_loss(*, trainer_logprobs: Tensor, inference_logprobs: Tensor, advantages: Tensor, loss_mask: Tensor,
                 rl_loss_fn, rl_scale: float, ce_scale: float = 1.0, ref_kl_scale: float = 1.0,
                 ref_logprobs: Tensor | None = None, rl_weights: Tensor | None = None,
                 ce_weights: Tensor | None = None, ref_kl_weights: Tensor | None = None,
                 sequence_lengths: list[int] | None = None) -> tuple[Tensor, dict[str, Tensor]]:
    """All inputs are flat ``[T]`` tensors of one packed micro-batch. Returns the scaled
    scalar loss (always connected to ``trainer_logprobs`` so every rank runs backward) and
    metric tensors."""
    metrics: dict[str, Tensor] = {}
    loss = trainer_logprobs.sum() * 0.0

    def run(fn, mask, weights, scale, per_sequence=False):
        nonlocal loss
        if per_sequence and sequence_lengths is not None:
            parts = zip(*(t.split(sequence_lengths) if t is not None else [None] * len(sequence_lengths)
                          for t in (trainer_logprobs, inference_logprobs, advantages, mask, ref_logprobs, weights)))
            outs = [fn(LossInputs(a, b, c, d, e, f)) for a, b, c, d, e, f in parts]
            total = sum(o.loss for o in outs)
            for k in outs[0].metrics:
                metrics[k] = torch.stack([o.metrics[k] for o in outs]).mean()
        else:
            out = fn(LossInputs(trainer_logprobs, inference_logprobs, advantages, mask, ref_logprobs, weights))
            total = out.loss
            metrics.update(out.metrics)
        loss = loss + total / scale

    rl_mask = loss_mask if rl_weights is None else loss_mask & (rl_weights != 0)
    run(rl_loss_fn.loss, rl_mask, rl_weights, rl_scale, per_sequence=getattr(rl_loss_fn, "per_sequence", False))
    if ce_weights is not None:
        run(ce_loss_fn, ce_weights != 0, ce_weights, ce_scale)
    if ref_kl_weights is not None:
        run(ref_kl_loss_fn, ref_kl_weights != 0, ref_kl_weights, ref_kl_scale)
    return loss, metrics
