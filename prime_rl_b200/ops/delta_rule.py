"""Gated delta rule (the linear-attention mixer of the Qwen3.5 / Qwen3-Next family) over packed
token streams.

Per head, with a state ``S [dk, dv]``, decay ``a_t = exp(g_t)``, write strength ``beta_t``, and
L2-normalised ``q, k``:

    S' = a_t S_{t-1}
    S_t = S' + beta_t k_t (v_t - k_t^T S')^T
    o_t = S_t^T q_t / sqrt(dk)

``gated_delta_rule`` evaluates it chunk-wise: inside a chunk the rank-one corrections are
resolved with one unit-lower-triangular solve (the "UT transform"), which turns the rest into
plain matrix products; between chunks only ``S`` is carried. The first token of every document
gets a log-decay of ``RESET`` (numerically zero), which clears the carried state at document
boundaries. ``gated_delta_rule_ref`` is the token-by-token recurrence for tests.

The reference calls ``fla.ops.gated_delta_rule.chunk_gated_delta_rule``
(src/prime_rl/trainer/models/qwen3_5/gated_delta_net.py:93-102).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .ssm import RESET


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.square().sum(-1, keepdim=True) + eps)


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                     position_ids: torch.Tensor, chunk: int = 64, l2norm: bool = True,
                     initial_state: torch.Tensor | None = None, return_state: bool = False):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g [T, H]`` (log-decay, <= 0), ``beta [T, H]``.
    Returns ``[T, H, dv]`` in fp32. ``initial_state [H, dk, dv]`` / ``return_state``: the state before the first and
    after the last token (serving: one sequence per call, continued across calls)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if l2norm:
        qf, kf = _l2norm(qf), _l2norm(kf)
    qf = qf * dk ** -0.5
    gf = torch.where((position_ids == 0).unsqueeze(1), torch.full_like(g.float(), RESET), g.float())
    bf = beta.float()
    C = chunk
    pad = (-T) % C

    def chunks(t):                                   # [T, H, ...] -> [H, nc, C, ...]
        if pad:
            t = F.pad(t, (0, 0) * (t.dim() - 1) + (0, pad))
        t = t.view((T + pad) // C, C, *t.shape[1:])
        return t.movedim(2, 0)

    qc, kc, vc = chunks(qf), chunks(kf), chunks(vf)                  # [H, nc, C, d]
    gc, bc = chunks(gf.unsqueeze(-1)).squeeze(-1), chunks(bf.unsqueeze(-1)).squeeze(-1)   # [H, nc, C]
    nc = qc.shape[1]
    cum = gc.cumsum(-1)                                              # decay from chunk start through token i
    diff = cum.unsqueeze(-1) - cum.unsqueeze(-2)                     # [H, nc, i, j]
    eye = torch.eye(C, dtype=torch.bool, device=q.device)
    lower = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    strict = lower & ~eye
    neg_inf = torch.full_like(diff, float("-inf"))
    decay_strict = torch.where(strict, diff, neg_inf).exp()
    decay_incl = torch.where(lower, diff, neg_inf).exp()
    kb = kc * bc.unsqueeze(-1)
    vb = vc * bc.unsqueeze(-1)
    # (I + A) u = rhs with A_ij = beta_i (k_i . k_j) exp(cum_i - cum_j), j < i
    Amat = (kb @ kc.transpose(-1, -2)) * decay_strict
    lhs = Amat + torch.eye(C, dtype=torch.float32, device=q.device)
    rhs = torch.cat([vb, kb * cum.exp().unsqueeze(-1)], dim=-1)
    sol = torch.linalg.solve_triangular(lhs, rhs, upper=False, unitriangular=True)
    u, w = sol[..., :dv], sol[..., dv:]                              # [H, nc, C, dv], [H, nc, C, dk]
    qk = (qc @ kc.transpose(-1, -2)) * decay_incl                    # [H, nc, C, C]
    k_to_end = kc * (cum[..., -1:] - cum).exp().unsqueeze(-1)
    end_decay = cum[..., -1].exp()                                   # [H, nc]
    q_in = qc * cum.exp().unsqueeze(-1)
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if initial_state is None \
        else initial_state.float()
    outs = []
    for c in range(nc):
        v_new = u[:, c] - w[:, c] @ S                                # what every token really writes
        outs.append(q_in[:, c] @ S + qk[:, c] @ v_new)
        S = S * end_decay[:, c, None, None] + k_to_end[:, c].transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=1)                                     # [H, nc, C, dv]
    o = o.movedim(0, 2).reshape(nc * C, H, dv)[:T]
    # padding tokens have g = 0, beta = 0 and k = 0: they neither decay nor write, so S is the state after token T - 1
    return (o, S) if return_state else o


def gated_delta_rule_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                          state: torch.Tensor, l2norm: bool = True):
    """One token for each of ``n`` sequences: ``q, k [n, H, dk]``, ``v [n, H, dv]``, ``g, beta [n, H]``,
    ``state [n, H, dk, dv]`` (fp32). Returns (o ``[n, H, dv]`` fp32, new state)."""
    dk = q.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if l2norm:
        qf, kf = _l2norm(qf), _l2norm(kf)
    qf = qf * dk ** -0.5
    state = state * g.float().exp()[:, :, None, None]
    pred = torch.einsum("bhk,bhkv->bhv", kf, state)
    state = state + beta.float()[:, :, None, None] * kf[..., None] * (vf - pred)[:, :, None, :]
    return torch.einsum("bhk,bhkv->bhv", qf, state), state


def gated_delta_rule_ref(q, k, v, g, beta, position_ids, l2norm: bool = True) -> torch.Tensor:
    T, H, dk = q.shape
    dv = v.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if l2norm:
        qf, kf = _l2norm(qf), _l2norm(kf)
    qf = qf * dk ** -0.5
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device)
    out = []
    for t in range(T):
        if int(position_ids[t]) == 0:
            S = torch.zeros_like(S)
        S = S * g[t].float().exp()[:, None, None]
        pred = torch.einsum("hk,hkv->hv", kf[t], S)
        S = S + beta[t].float()[:, None, None] * kf[t][:, :, None] * (vf[t] - pred)[:, None, :]
        out.append(torch.einsum("hk,hkv->hv", qf[t], S))
    return torch.stack(out)
