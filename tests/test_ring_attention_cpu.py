"""Block form of attention used by the ring style of context parallelism: partial results over key ranges merge to
the full result, and the block backward (given the final output and log-sum-exp) sums to the full gradients."""

import math

import pytest
import torch

from prime_rl_b200.parallel import ring_attn


def _full(q, k, v, cu, window=None):
    T, Hq, D = q.shape
    g = Hq // k.shape[1]
    pos = torch.arange(T)
    doc = torch.searchsorted(cu[1:].contiguous(), pos, right=True)
    mask = (doc[:, None] == doc[None, :]) & (pos[None, :] <= pos[:, None])
    if window:
        mask &= pos[:, None] - pos[None, :] < window
    s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(g, 1)) / math.sqrt(D)
    p = torch.softmax(s.masked_fill(~mask[None], float("-inf")), -1)
    return torch.einsum("hts,shd->thd", p, v.repeat_interleave(g, 1))


@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("chunks", [2, 4, 8])
def test_partial_blocks_merge_to_full_attention_and_gradients(chunks, window):
    torch.manual_seed(0)
    T, Hq, Hkv, D = 128, 4, 2, 16
    cu = torch.tensor([0, 50, 51, 128])
    q, k, v = (torch.randn(T, h, D, dtype=torch.float64, requires_grad=True) for h in (Hq, Hkv, Hkv))
    ref = _full(q, k, v, cu, window)
    dout = torch.randn_like(ref)
    dq_ref, dk_ref, dv_ref = torch.autograd.grad(ref, (q, k, v), dout)

    c = T // chunks
    acc = torch.zeros(T, Hq, D, dtype=torch.float32)
    lse = torch.full((Hq, T), float("-inf"))
    qd, kd, vd = q.detach().float(), k.detach().float(), v.detach().float()
    for qi in range(chunks):
        a, l = acc[qi * c:(qi + 1) * c], lse[:, qi * c:(qi + 1) * c].clone()
        for ki in range(chunks):                       # also the blocks above the diagonal: they must come back empty
            part, lp, _ = ring_attn.block_fwd_ref(qd[qi * c:(qi + 1) * c], kd[ki * c:(ki + 1) * c], vd[ki * c:(ki + 1) * c],
                                                  cu, T, qi * c, ki * c, window)
            if ki > qi:
                assert torch.isinf(lp).all() and part.abs().max() == 0
            ring_attn.merge_partial(a, l, part, lp)
        lse[:, qi * c:(qi + 1) * c] = l
    torch.testing.assert_close(acc.double(), ref.detach(), atol=2e-5, rtol=1e-4)

    dq, dk, dv = torch.zeros_like(qd), torch.zeros_like(kd), torch.zeros_like(vd)
    for qi in range(chunks):
        for ki in range(qi + 1):
            rows, keys = slice(qi * c, (qi + 1) * c), slice(ki * c, (ki + 1) * c)
            a, b, e = ring_attn._block_bwd(dout[rows].float(), qd[rows], kd[keys], vd[keys], acc[rows], lse[:, rows], cu, T,
                                           qi * c, ki * c, window)
            dq[rows] += a
            dk[keys] += b
            dv[keys] += e
    torch.testing.assert_close(dq.double(), dq_ref, atol=5e-5, rtol=1e-3)
    torch.testing.assert_close(dk.double(), dk_ref, atol=5e-5, rtol=1e-3)
    torch.testing.assert_close(dv.double(), dv_ref, atol=5e-5, rtol=1e-3)


def test_ring_pairs_are_balanced_in_the_zigzag_layout():
    class CP:
        layout = "zigzag"

    for cp in (2, 4, 8):
        counts = []
        for rank in range(cp):
            c = CP()
            c.cp, c.rank = cp, rank
            per_step = [len(ring_attn._pairs(c, (rank - s) % cp, 64, None)) for s in range(cp)]
            assert per_step[0] == 3 and all(n == 2 for n in per_step[1:])
            counts.append(sum(per_step))
        assert len(set(counts)) == 1


@pytest.mark.slow
def test_ring_attention_on_four_cpu_ranks_matches_the_all_gather_path(free_port):
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(root))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port), "-m", "tests.distributed.ring_attention_cpu"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0 and "RING_CPU_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
