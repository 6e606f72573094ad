import math

import torch

from prime_rl_b200.configs.trainer import IcePopLossConfig, IPOLossConfig
from prime_rl_b200.trainer.loss import (IcePopLoss, IPOLoss, LossInputs, ce_loss_fn, compute_loss, ref_kl_loss_fn,
                                        setup_rl_loss_fn, shift_left, shift_right)


def _inputs(n=64):
    g = torch.Generator().manual_seed(0)
    lp = (-torch.rand(n, generator=g) * 2).requires_grad_()
    old = lp.detach() + 0.05 * torch.randn(n, generator=g)
    adv = torch.randn(n, generator=g)
    mask = torch.rand(n, generator=g) > 0.3
    return lp, old, adv, mask


def test_shift_helpers():
    t = torch.arange(6.0)
    assert shift_left(t).tolist() == [1, 2, 3, 4, 5, 0]
    assert shift_right(t, -1.0).tolist() == [-1, 0, 1, 2, 3, 4]
    t2 = torch.arange(6.0).view(1, 6)
    assert shift_left(t2).tolist() == [[1, 2, 3, 4, 5, 0]]


def test_ipo_matches_formula_and_grad():
    lp, old, adv, mask = _inputs()
    cfg = IPOLossConfig()
    out = IPOLoss(cfg).loss(LossInputs(lp, old, adv, mask))
    ratio = torch.exp(lp - old)
    keep = mask & ((torch.exp(lp) - torch.exp(old)).abs() <= cfg.eps)
    want = (-(keep * adv * ratio) + cfg.kl_tau * mask * (lp - old) ** 2).sum()
    assert torch.allclose(out.loss, want, atol=1e-6)
    out.loss.backward()
    g = lp.grad
    want_g = -(keep * adv * ratio) + 2 * cfg.kl_tau * mask * (lp - old)
    assert torch.allclose(g, want_g.detach(), atol=1e-6)
    assert 0.0 <= out.metrics["is_masked"] <= 1.0


def test_icepop_band_and_no_nan():
    lp, old, adv, mask = _inputs()
    old = old.clone()
    old[0] = lp.detach()[0] - 100.0  # absurd ratio must be masked, not NaN
    out = IcePopLoss(IcePopLossConfig()).loss(LossInputs(lp, old, adv, mask | True))
    out.loss.backward()
    assert torch.isfinite(out.loss) and torch.isfinite(lp.grad).all() and lp.grad[0] == 0


def test_components_and_global_scales():
    lp, old, adv, mask = _inputs()
    ref = old + 0.1
    ce_w = torch.zeros_like(old)
    ce_w[:10] = 2.0
    rk_w = torch.zeros_like(old)
    rk_w[10:20] = 1.0
    fn = setup_rl_loss_fn(IPOLossConfig())
    loss, metrics = compute_loss(trainer_logprobs=lp, inference_logprobs=old, advantages=adv, loss_mask=mask,
                                 rl_loss_fn=fn, rl_scale=40.0, ce_scale=10.0, ref_kl_scale=5.0, ref_logprobs=ref,
                                 ce_weights=ce_w, ref_kl_weights=rk_w)
    rl = fn.loss(LossInputs(lp, old, adv, mask)).loss / 40.0
    ce = ce_loss_fn(LossInputs(lp, old, adv, ce_w != 0, None, ce_w)).loss / 10.0
    rk = ref_kl_loss_fn(LossInputs(lp, old, adv, rk_w != 0, ref, rk_w)).loss / 5.0
    assert torch.allclose(loss, rl + ce + rk, atol=1e-6)
    assert "nll" in metrics and "ref_kl" in metrics


def test_empty_mask_still_backpropagates():
    lp, old, adv, mask = _inputs()
    loss, _ = compute_loss(trainer_logprobs=lp, inference_logprobs=old, advantages=adv,
                           loss_mask=torch.zeros_like(mask), rl_loss_fn=setup_rl_loss_fn(IPOLossConfig()),
                           rl_scale=1.0)
    loss.backward()
    assert lp.grad is not None and float(loss) == 0.0 and math.isfinite(float(loss))
