"""Sequence mixers with a recurrent state over packed token streams: the depthwise causal
convolution and the Mamba-2 selective state-space scan (SSD).

Documents of a packed micro-batch must not see each other. Both ops take the per-token
position inside its document (``position_ids``): the convolution masks taps that would reach
before a document's first token, and the scan gives a document's first token a decay of
``exp(RESET)`` (numerically zero), which clears the carried state exactly where the recurrence
``S_t = a_t S_{t-1} + dt_t x_t B_t^T`` would otherwise leak it.

The scan is the chunked SSD algorithm: inside a chunk of Q tokens the output is a masked,
decay-weighted ``(C B^T) x`` product (tensor-core shaped), between chunks a small state
``[heads, head_dim, state]`` is carried. ``mamba2_scan_ref`` is the token-by-token recurrence
used by the tests.

The reference calls ``fla.modules.conv.causal_conv1d`` and
``mamba_ssm.ops.triton.ssd_combined.mamba_chunk_scan_combined`` for these
(src/prime_rl/trainer/models/nemotron_h/mamba.py:81-83, :201-236).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

RESET = -80.0      # log-decay given to the first token of a document: exp(-80) ~ 1.8e-35


class _CausalConv1d(torch.autograd.Function):
    """``csrc/conv1d.cu``: bf16, 8 channels per thread, document boundaries from ``position_ids``."""

    @staticmethod
    def forward(ctx, x, weight, bias, pos, silu):
        from . import _runtime as rt

        T, C = x.shape
        y = torch.empty_like(x)
        rt.check(rt.lib().prb_conv1d_fwd(x.data_ptr(), weight.data_ptr(), rt.ptr(bias), pos.data_ptr(), y.data_ptr(), T, C,
                                         weight.shape[1], int(silu), rt.stream_ptr(x.device)), "prb_conv1d_fwd")
        ctx.save_for_backward(x, weight, bias, pos)
        ctx.silu = silu
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _runtime as rt

        x, weight, bias, pos = ctx.saved_tensors
        T, C = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(C, weight.shape[1], dtype=torch.float32, device=x.device)
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if bias is not None else None
        rt.check(rt.lib().prb_conv1d_bwd(x.data_ptr(), weight.data_ptr(), rt.ptr(bias), pos.data_ptr(), dy.data_ptr(),
                                         dx.data_ptr(), dw.data_ptr(), rt.ptr(db), T, C, weight.shape[1], int(ctx.silu),
                                         rt.stream_ptr(x.device)), "prb_conv1d_bwd")
        return dx, dw.to(weight.dtype), (db.to(bias.dtype) if db is not None else None), None, None


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, position_ids: torch.Tensor,
                  activation: str | None = "silu") -> torch.Tensor:
    """Depthwise causal convolution over tokens. ``x [T, C]``, ``weight [C, K]`` (tap K-1 multiplies
    the current token), ``position_ids [T]`` position of every token in its document."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and weight.shape[1] <= 4 and activation in ("silu", "swish", None)
            and (bias is None or bias.dtype == torch.bfloat16)):
        return _CausalConv1d.apply(x.contiguous(), weight.contiguous(), bias, position_ids.to(torch.int32).contiguous(),
                                   activation is not None)
    return causal_conv1d_ref(x, weight, bias, position_ids, activation)


def causal_conv1d_ref(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, position_ids: torch.Tensor,
                      activation: str | None = "silu") -> torch.Tensor:
    """PyTorch definition of ``causal_conv1d`` (CPU path and oracle of the kernel)."""
    T, C = x.shape
    K = weight.shape[1]
    xf = x.float()
    y = xf * weight[:, K - 1].float()
    for s in range(1, K):
        if s >= T:
            break
        shifted = F.pad(xf[:-s], (0, 0, s, 0))
        ok = (position_ids >= s).unsqueeze(1)
        y = y + torch.where(ok, shifted, torch.zeros((), dtype=xf.dtype, device=x.device)) * weight[:, K - 1 - s].float()
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    elif activation is not None:
        raise ValueError(f"unsupported activation '{activation}'")
    return y.to(x.dtype)


def _pad_tokens(t: torch.Tensor, n: int) -> torch.Tensor:
    if n == 0:
        return t
    return F.pad(t, (0, 0) * (t.dim() - 1) + (0, n))


def mamba2_scan(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor,
                D: torch.Tensor | None, position_ids: torch.Tensor, chunk: int = 128,
                initial_state: torch.Tensor | None = None, return_state: bool = False):
    """Chunked SSD. ``x [T, H, P]``, ``dt [T, H]`` (after softplus / clamping), ``A [H]`` (negative),
    ``B, C [T, G, N]`` with ``H % G == 0``, ``D [H]`` skip weight. Returns ``[T, H, P]`` in fp32.
    ``initial_state [H, P, N]``: the state before the first token (a sequence continued from an earlier call: its
    positions then do not start at 0). ``return_state``: also return the state after the last token (serving:
    one sequence per call)."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    Q = chunk
    pad = (-T) % Q
    xf, dtf = _pad_tokens(x.float(), pad), _pad_tokens(dt.float(), pad)
    Bf, Cf = _pad_tokens(B.float(), pad), _pad_tokens(C.float(), pad)
    pos = F.pad(position_ids, (0, pad), value=1)
    a = dtf * A.float()                                              # [Tp, H] log-decay per token
    a = torch.where((pos == 0).unsqueeze(1), torch.full_like(a, RESET), a)
    nc = (T + pad) // Q
    xc = xf.view(nc, Q, H, P)
    dtc = dtf.view(nc, Q, H)
    ac = a.view(nc, Q, H)
    Bc = Bf.view(nc, Q, G, N)
    Cc = Cf.view(nc, Q, G, N)
    cum = ac.cumsum(1)                                               # inclusive: decay from chunk start through token i
    # ---- inside a chunk: y_i += sum_{j <= i} exp(cum_i - cum_j) dt_j (C_i . B_j) x_j
    diff = cum.unsqueeze(2) - cum.unsqueeze(1)                       # [nc, Q(i), Q(j), H]
    tri = torch.ones(Q, Q, dtype=torch.bool, device=x.device).tril()
    L = torch.where(tri[None, :, :, None], diff, torch.full_like(diff, float("-inf"))).exp()
    cb = torch.einsum("cign,cjgn->cijg", Cc, Bc)                     # [nc, Q, Q, G]
    M = L * dtc.unsqueeze(1) * cb.repeat_interleave(rep, dim=3)      # [nc, Q, Q, H]
    y = torch.einsum("cijh,cjhp->cihp", M, xc)
    # ---- state every chunk hands on: sum_j exp(cum_end - cum_j) dt_j x_j B_j^T
    to_end = (cum[:, -1:, :] - cum).exp() * dtc                      # [nc, Q, H]
    Bh = Bc.repeat_interleave(rep, dim=2)                            # [nc, Q, H, N]
    Ch = Cc.repeat_interleave(rep, dim=2)
    S_chunk = torch.einsum("cjh,cjhp,cjhn->chpn", to_end, xc, Bh)
    chunk_decay = cum[:, -1, :].exp()                                # [nc, H]
    # ---- carry between chunks (a short sequential loop over nc small tensors)
    carry = torch.zeros(H, P, N, dtype=torch.float32, device=x.device) if initial_state is None \
        else initial_state.float()
    carries = []
    for c in range(nc):
        carries.append(carry)
        carry = carry * chunk_decay[c][:, None, None] + S_chunk[c]
    S_in = torch.stack(carries)                                      # state entering every chunk
    y = y + torch.einsum("cih,cihn,chpn->cihp", cum.exp(), Ch, S_in)
    y = y.reshape(nc * Q, H, P)[:T]
    if D is not None:
        y = y + x.float() * D.float()[None, :, None]
    # padding tokens have dt = 0: no decay and no contribution, so the carry after the last chunk is the state
    # after token T - 1
    return (y, carry) if return_state else y


def mamba2_step(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor,
                D: torch.Tensor | None, state: torch.Tensor):
    """One token for each of ``n`` sequences: ``x [n, H, P]``, ``dt [n, H]``, ``B, C [n, G, N]``, ``state [n, H, P, N]``
    (fp32). Returns (y ``[n, H, P]`` fp32, new state)."""
    H, G = x.shape[1], B.shape[1]
    rep = H // G
    dA = (dt.float() * A.float()).exp()                                   # [n, H]
    Bh = B.float().repeat_interleave(rep, dim=1)                          # [n, H, N]
    Ch = C.float().repeat_interleave(rep, dim=1)
    state = state * dA[:, :, None, None] + (dt.float()[:, :, None] * x.float())[..., None] * Bh[:, :, None, :]
    y = torch.einsum("bhpn,bhn->bhp", state, Ch)
    if D is not None:
        y = y + x.float() * D.float()[None, :, None]
    return y, state


def conv1d_window(tail: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                  activation: str | None = "silu"):
    """Causal convolution of the new tokens of ONE sequence whose last ``K - 1`` inputs are ``tail [K - 1, C]``
    (zeros before the first token). Returns (y ``[n, C]``, new tail)."""
    K = weight.shape[1]
    full = torch.cat([tail.to(x.dtype), x], 0)
    pos = torch.arange(K, K + full.shape[0], dtype=torch.int32, device=x.device)      # no tap is masked
    y = causal_conv1d(full, weight, bias, pos, activation)[K - 1:]
    return y, full[full.shape[0] - (K - 1):]


def conv1d_step(tails: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                activation: str | None = "silu"):
    """One token for each of ``n`` sequences: ``tails [n, K - 1, C]``, ``x [n, C]``. Returns (y ``[n, C]``, new tails)."""
    win = torch.cat([tails.to(x.dtype), x[:, None, :]], 1)                # [n, K, C]
    y = torch.einsum("nkc,ck->nc", win.float(), weight.float())
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype), win[:, 1:]


def mamba2_scan_ref(x, dt, A, B, C, D, position_ids) -> torch.Tensor:
    """Token-by-token recurrence (fp32), for tests."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    S = torch.zeros(H, P, N, dtype=torch.float32, device=x.device)
    out = []
    for t in range(T):
        if int(position_ids[t]) == 0:
            S = torch.zeros_like(S)
        dA = (dt[t].float() * A.float()).exp()
        Bt = B[t].float().repeat_interleave(rep, dim=0)
        Ct = C[t].float().repeat_interleave(rep, dim=0)
        S = S * dA[:, None, None] + dt[t].float()[:, None, None] * x[t].float()[:, :, None] * Bt[:, None, :]
        y = torch.einsum("hpn,hn->hp", S, Ct)
        if D is not None:
            y = y + x[t].float() * D.float()[:, None]
        out.append(y)
    return torch.stack(out)


class _GatedNorm(torch.autograd.Function):
    """``csrc/gated_norm.cu``: one warp per (row, group); dw summed in registers per warp."""

    @staticmethod
    def forward(ctx, x, gate, weight, eps, group, gate_first):
        from . import _runtime as rt

        rows, cols = x.shape
        y = torch.empty_like(x)
        rt.check(rt.lib().prb_gated_norm_fwd(x.data_ptr(), gate.data_ptr(), weight.data_ptr(), y.data_ptr(), rows, cols,
                                             group, weight.numel(), float(eps), int(gate_first), rt.stream_ptr(x.device)),
                 "prb_gated_norm_fwd")
        ctx.save_for_backward(x, gate, weight)
        ctx.cfg = (eps, group, gate_first)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _runtime as rt

        x, gate, weight = ctx.saved_tensors
        eps, group, gate_first = ctx.cfg
        rows, cols = x.shape
        dy = dy.contiguous()
        dx, dg = torch.empty_like(x), torch.empty_like(gate)
        dw = torch.zeros(weight.numel(), dtype=torch.float32, device=x.device)
        rt.check(rt.lib().prb_gated_norm_bwd(x.data_ptr(), gate.data_ptr(), weight.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                             dg.data_ptr(), dw.data_ptr(), rows, cols, group, weight.numel(), float(eps),
                                             int(gate_first), rt.stream_ptr(x.device)), "prb_gated_norm_bwd")
        return dx, dg, dw.to(weight.dtype), None, None, None


def gated_rms_norm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, group_size: int,
                   gate_act: str = "silu", gate_first: bool = True) -> torch.Tensor:
    """RMSNorm over groups of ``group_size`` channels combined with a gate. ``gate_first``:
    ``norm(x * act(gate)) * w`` (Mamba-2); otherwise ``norm(x) * w * act(gate)`` (gated delta-net).
    ``weight`` has one entry per channel of the last dim, or ``group_size`` entries shared by all groups."""
    cols = x.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and gate_act in ("silu", "swish") and group_size % 8 == 0 and group_size <= 1024
            and weight.numel() in (cols, group_size) and weight.numel() % 8 == 0):
        shp = x.shape
        y = _GatedNorm.apply(x.reshape(-1, cols).contiguous(), gate.reshape(-1, cols).contiguous(), weight.contiguous(),
                             eps, group_size, gate_first)
        return y.reshape(shp)
    return gated_rms_norm_ref(x, gate, weight, eps, group_size, gate_act, gate_first)


def gated_rms_norm_ref(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, group_size: int,
                       gate_act: str = "silu", gate_first: bool = True) -> torch.Tensor:
    """PyTorch definition of ``gated_rms_norm`` (CPU path and oracle of the kernel)."""
    act = F.silu if gate_act in ("silu", "swish") else torch.sigmoid
    xf = x.float()
    if gate_first:
        xf = xf * act(gate.float())
    shp = xf.shape
    g = xf.reshape(*shp[:-1], shp[-1] // group_size, group_size)
    g = g * torch.rsqrt(g.square().mean(-1, keepdim=True) + eps)
    y = g.reshape(shp) * weight.float()
    if not gate_first:
        y = y * act(gate.float())
    return y.to(x.dtype)
