import pytest
import torch

from prime_rl_b200.native import build as nb
from prime_rl_b200.ops import cpu_optim


@pytest.fixture(scope="module", autouse=True)
def _built():
    nb.build_cpu()


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("odtype", [None, torch.bfloat16, torch.float32])
def test_cpu_adamw_matches_torch(gdtype, odtype):
    n = 100_003
    p = torch.randn(n)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(n), torch.zeros(n)
    out = torch.empty(n, dtype=odtype) if odtype is not None else None
    for step in range(1, 4):
        g = torch.randn(n).to(gdtype)
        ref.grad = g.float() * 0.5
        opt.step()
        cpu_optim.cpu_adamw_step(p, m, v, g, out, step=step, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1,
                                 grad_scale=0.5)
    assert torch.allclose(p, ref.detach(), atol=1e-6, rtol=1e-5)
    if out is not None:
        assert torch.allclose(out.float(), p, atol=1e-2 if odtype == torch.bfloat16 else 0, rtol=1e-2)


def test_cpu_sign_sgd_and_bf16_accumulate():
    n = 70_001
    p, g = torch.randn(n), torch.randn(n)
    g[::5] = 0
    want = p + p * (-1e-2 * 0.1) + torch.sign(g) * (-1e-2)
    out = torch.empty(n, dtype=torch.bfloat16)
    cpu_optim.cpu_sign_sgd_step(p, g, out, lr=1e-2, wd=0.1)
    assert torch.allclose(p, want, atol=1e-7) and torch.allclose(out.float(), want, atol=2e-2, rtol=1e-2)
    acc = torch.ones(n)
    src = torch.randn(n).bfloat16()
    cpu_optim.bf16_to_fp32_(acc, src, accumulate=True)
    assert torch.equal(acc, 1 + src.float())
    cpu_optim.bf16_to_fp32_(acc, src)
    assert torch.equal(acc, src.float())
