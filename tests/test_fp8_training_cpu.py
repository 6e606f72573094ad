"""fp8 training path on CPU (the quantisers and the block-scaled product have PyTorch references): the fp8 linear and
grouped linear stay within e4m3 accuracy of the exact products, weight copies are refreshed per optimizer step, and a
trainer with ``model.quantization = fp8`` follows the unquantised run."""

import json

import pytest
import torch

from prime_rl_b200.ops import fp8 as F


def _rel(a, b):
    return float((a.detach().float() - b.detach().float()).norm() / b.detach().float().norm())


def test_fp8_linear_forward_and_input_gradient_are_close_and_weight_gradient_is_exact():
    torch.manual_seed(0)
    x = torch.randn(70, 256, requires_grad=True)
    w = (torch.randn(384, 256) * 0.05).requires_grad_()
    b = torch.randn(384)
    y = F.fp8_linear(x, w, b)
    ref = x @ w.t() + b
    assert _rel(y, ref) < 0.06
    dy = torch.randn_like(ref)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    rx, rw = torch.autograd.grad(ref, (x, w), dy)
    assert _rel(gx, rx) < 0.06
    assert _rel(gw, rw) < 1e-5            # the weight gradient is not quantised


def test_fp8_grouped_linear_matches_per_expert_products():
    torch.manual_seed(1)
    E, N, K = 3, 128, 256
    block_expert = torch.tensor([0, 0, 2, 1, -1], dtype=torch.int32)
    expert_offset = torch.tensor([0, 256, 384, 512], dtype=torch.int32)
    # rows are laid out in block order: blocks 0, 1 -> expert 0; block 2 -> expert 2; block 3 -> expert 1; block 4 unused
    x = torch.randn(640, K, requires_grad=True)
    w = (torch.randn(E, N, K) * 0.05).requires_grad_()
    y = F._FP8GroupedLinear.apply(x, w, block_expert, expert_offset)
    ref = torch.zeros(640, N)
    for blk, e in enumerate(block_expert.tolist()):
        if e >= 0:
            ref[blk * 128:(blk + 1) * 128] = x[blk * 128:(blk + 1) * 128].detach() @ w[e].detach().t()
    assert _rel(y[:512], ref[:512]) < 0.06
    assert float(y[512:].detach().abs().max()) == 0.0
    dy = torch.randn(640, N)
    dy[512:] = 0
    (gx,) = torch.autograd.grad(y, (x,), dy)
    rx = torch.zeros_like(x)
    for blk, e in enumerate(block_expert.tolist()):
        if e >= 0:
            rx[blk * 128:(blk + 1) * 128] = dy[blk * 128:(blk + 1) * 128] @ w[e].detach()
    assert _rel(gx[:512], rx[:512]) < 0.06


def test_weight_copies_are_cached_per_optimizer_step():
    torch.manual_seed(2)
    w = torch.randn(128, 128)
    F.bump_weight_epoch()
    a = F.weight_fp8(w, False)
    assert F.weight_fp8(w, False)[0] is a[0]                 # same step: the copy is reused
    t = F.weight_fp8(w, True)
    assert torch.equal(t[0].view(torch.float8_e4m3fn).float().t(), a[0].view(torch.float8_e4m3fn).float())
    w.mul_(2.0)
    F.bump_weight_epoch()
    b = F.weight_fp8(w, False)
    assert b[0] is not a[0] and torch.allclose(b[1], a[1] * 2)


@pytest.mark.slow
def test_trainer_with_fp8_projections_follows_the_unquantised_run(tmp_path):
    from prime_rl_b200.configs.trainer import TrainerConfig
    from prime_rl_b200.trainer.rl.train import RLTrainer

    def run(quant):
        torch.manual_seed(0)
        cfg = {"model": {"name": "tiny-qwen3-moe", "seq_len": 256, "ep": 1, "ac": None, "debug": {"random_init": True}},
               "data": {"fake": {"batch_size": 2}}, "optim": {"lr": 1e-3, "max_norm": 1.0}, "monitors": {"file": None},
               "output_dir": str(tmp_path / ("q" if quant else "b"))}
        if quant:
            cfg["model"]["quantization"] = {"type": "fp8"}
        tr = RLTrainer(TrainerConfig.model_validate(json.loads(json.dumps(cfg)))).setup()
        flagged = [n for n, m in tr.model.named_modules() if getattr(m, "fp8_train", False)]
        out = []
        for _ in range(3):
            m = tr.step()
            out.append((m["loss"], m["optim/grad_norm"], m["entropy"]))
        return out, flagged

    base, none = run(False)
    quant, flagged = run(True)
    assert not none and any("experts" in n for n in flagged) and any("qkv_proj" in n for n in flagged)
    assert not any("lm_head" in n or n.endswith("router") or n.endswith("mlp.gate") for n in flagged)
    for (l0, g0, e0), (l1, g1, e1) in zip(base, quant):
        assert e1 == pytest.approx(e0, rel=2e-2)
        assert g1 == pytest.approx(g0, rel=0.25)
        assert l1 == pytest.approx(l0, abs=5e-3)


def test_fp8_weight_gradient_option():
    torch.manual_seed(4)
    x = torch.randn(64, 256, requires_grad=True)
    w = (torch.randn(384, 256) * 0.05).requires_grad_()
    dy = torch.randn(64, 384)
    (rw,) = torch.autograd.grad(x @ w.t(), (w,), dy)
    F.FP8_WGRAD = True
    try:
        (gw,) = torch.autograd.grad(F.fp8_linear(x, w), (w,), dy)
    finally:
        F.FP8_WGRAD = False
    rel = _rel(gw, rw)
    assert 1e-4 < rel < 0.06            # quantised, and within e4m3 accuracy
