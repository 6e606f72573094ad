import math

import pytest

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


def test_sampling_mask_replay_matches_masked_log_softmax():
    import torch
    from prime_rl_b200 import ops

    torch.manual_seed(0)
    T, H, V, K = 23, 16, 50, 6
    h = torch.randn(T, H, requires_grad=True)
    w = torch.randn(V, H) * 0.3
    labels = torch.randint(0, V, (T,))
    inv_t = torch.rand(T) + 0.5
    mask = torch.full((T, K), -1, dtype=torch.int32)
    for t in range(T):
        if t % 5 == 0:
            continue                                        # empty mask: full-vocabulary value
        ids = torch.randperm(V)[: (t % K) + 1]
        if t % 7 != 0:
            ids[0] = labels[t]                              # t % 7 == 0: label not in mask -> full vocabulary
        mask[t, : len(ids)] = ids.to(torch.int32)
    full, _ = ops.logprob_entropy_ref(h, w, labels, inv_t)
    got = ops.replay_sampling_mask(full, h, w, labels, inv_t, mask, bytes_budget=4 * K * H * 4)
    z = (h @ w.t()) * inv_t[:, None]
    for t in range(T):
        ids = [int(i) for i in mask[t] if int(i) >= 0]
        if ids and int(labels[t]) in ids:
            want = z[t, labels[t]] - torch.logsumexp(z[t, ids], 0)
        else:
            want = full[t]
        assert abs(float(got[t] - want)) < 1e-5, t
    got.sum().backward()
    assert torch.isfinite(h.grad).all()


def test_softcapped_head_matches_direct_formula():
    import torch
    from prime_rl_b200 import ops

    torch.manual_seed(1)
    T, H, V = 19, 8, 40
    h = torch.randn(T, H, requires_grad=True)
    w = torch.randn(V, H)
    labels = torch.randint(0, V, (T,))
    lp, ent = ops.softcapped_logprob_entropy(h, w, labels, None, softcap=5.0, chunk=7)
    z = 5.0 * torch.tanh((h @ w.t()) / 5.0)
    want = torch.log_softmax(z, -1).gather(1, labels[:, None]).squeeze(1)
    assert torch.allclose(lp, want, atol=1e-5)
    p = torch.softmax(z, -1)
    assert torch.allclose(ent, -(p * torch.log(p)).sum(-1), atol=1e-4)
    g1, = torch.autograd.grad(lp.sum(), h, retain_graph=True)
    g2, = torch.autograd.grad(want.sum(), h)
    assert torch.allclose(g1, g2, atol=1e-5)


def test_token_statistics_match_torch_on_the_concatenated_values():
    """mean / median / std / min / max from sufficient statistics and histogram bisection equal the direct
    computation on all values (single process; the multi-rank reduction is covered by the gloo tests)."""
    from prime_rl_b200.trainer.stats import TensorStats

    g = torch.Generator().manual_seed(3)
    for n in (1, 2, 7, 4097, 20000):
        x = torch.randn(n, generator=g) * 5 - 2
        x[::3] = x[0]                                      # ties
        st = TensorStats()
        st.add("x", x[: n // 2])
        st.add("x", x[n // 2:], mask=torch.ones(n - n // 2, dtype=torch.bool))
        st.add("none", torch.empty(0))
        out = st.compute()
        assert out["x/median"].item() == x.median().item()
        assert out["x/min"].item() == x.min().item() and out["x/max"].item() == x.max().item()
        assert out["x/mean"].item() == pytest.approx(x.mean().item(), rel=1e-5, abs=1e-6)
        if n > 1:
            assert out["x/std"].item() == pytest.approx(x.std().item(), rel=1e-4)
        assert out["none/mean"].item() != out["none/mean"].item()      # NaN for an empty key
    assert st.values == {}
