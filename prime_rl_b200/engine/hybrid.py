"""Rollout runner for the families whose layers carry a recurrent state (Mamba-2 blocks of Nemotron-H, gated
delta-net layers of Qwen3.5 / Qwen3.5-MoE) next to softmax attention.

The model's own ``forward`` runs unchanged; a ``RecurrentStep`` object rides on ``SeqInfo.engine`` and the mixers hand
it the three operations whose meaning depends on what came before the new tokens:

  ``attend``   softmax attention (``Attention``, ``GatedAttention``): the new K / V go into the paged cache, then the new
               queries attend the cached prefix + themselves (paged decode kernel for one-token steps on a GPU)
  ``conv``     the depthwise causal convolution: every sequence keeps its last ``K - 1`` inputs per layer
  ``mamba`` / ``delta``  the state-space scan and the gated delta rule: every sequence keeps the state ``[H, P, N]`` /
               ``[H, dk, dv]`` per layer (fp32); a prefill (or a chunk of one) runs the chunked scan from the stored
               state and stores the state after its last token; a decode step runs one batched recurrence step for
               all sequences

The state lives on the request's ``SequenceKV`` object, so it is dropped together with the pages when a request
finishes or is preempted (a preempted request recomputes from its tokens). A recurrent state cannot be shared
through the page-level prefix cache, so engines of these families run without it.

The reference serves these families through vLLM's hybrid KV-cache manager (one Mamba state slot per request next to
the attention pages); its own code only configures it (packages/prime-rl-configs/src/prime_rl/configs/inference.py).
"""

from __future__ import annotations

import torch

from ..models.layers import SeqInfo
from ..ops import delta_rule, ssm
from .runner import ModelRunner, StepInput


class RecurrentStep:
    def __init__(self, runner: "HybridRunner", batch: list[StepInput], starts: list[int], slots_t: torch.Tensor):
        self.runner, self.batch, self.starts, self.slots = runner, batch, starts, slots_t
        self.lens = [len(s.tokens) for s in batch]
        self.decode = all(n == 1 and s.kv.length > 0 for n, s in zip(self.lens, batch))
        for s in batch:
            if s.kv.length == 0 or getattr(s.kv, "mixer_state", None) is None:
                s.kv.mixer_state = {}               # a fresh (or restarted) sequence starts from nothing

    # ---------------------------------------------------------------- state bookkeeping
    def _get(self, s: StepInput, key, shape, dtype, device):
        st = s.kv.mixer_state
        t = st.get(key)
        if t is None:
            t = torch.zeros(shape, dtype=dtype, device=device)
            st[key] = t
        return t

    # ---------------------------------------------------------------- attention
    def attend(self, layer: int, q, k, v, window, sinks):
        cache = self.runner.cache
        Hkv, D = k.shape[1], k.shape[2]
        cache.k[layer].view(-1, Hkv, D).index_copy_(0, self.slots, k.to(cache.k.dtype))
        cache.v[layer].view(-1, Hkv, D).index_copy_(0, self.slots, v.to(cache.v.dtype))
        return self.runner._attend(layer, q, k, v, self.batch, self.starts, window, sinks)

    # ---------------------------------------------------------------- convolution
    def conv(self, layer: int, x, weight, bias, activation="silu"):
        K, C = weight.shape[1], x.shape[1]
        key = (layer, "conv")
        tails = [self._get(s, key, (K - 1, C), x.dtype, x.device) for s in self.batch]
        if self.decode:
            y, new = ssm.conv1d_step(torch.stack(tails), x, weight, bias, activation)
            for s, t in zip(self.batch, new):
                s.kv.mixer_state[key] = t
            return y
        outs = []
        for s, st, n, tail in zip(self.batch, self.starts, self.lens, tails):
            y, new = ssm.conv1d_window(tail, x[st:st + n], weight, bias, activation)
            s.kv.mixer_state[key] = new
            outs.append(y)
        return torch.cat(outs, 0)

    # ---------------------------------------------------------------- Mamba-2
    def mamba(self, layer: int, x, dt, A, B, C, D, chunk: int):
        H, P, N = x.shape[1], x.shape[2], B.shape[2]
        key = (layer, "ssm")
        states = [self._get(s, key, (H, P, N), torch.float32, x.device) for s in self.batch]
        if self.decode:
            y, new = ssm.mamba2_step(x, dt, A, B, C, D, torch.stack(states))
            for s, t in zip(self.batch, new):
                s.kv.mixer_state[key] = t
            return y
        outs = []
        for s, st, n, state in zip(self.batch, self.starts, self.lens, states):
            pos = torch.arange(s.kv.length, s.kv.length + n, dtype=torch.int32, device=x.device)
            sl = slice(st, st + n)
            y, new = ssm.mamba2_scan(x[sl], dt[sl], A, B[sl], C[sl], D, pos, chunk=chunk,
                                     initial_state=state if s.kv.length else None, return_state=True)
            s.kv.mixer_state[key] = new
            outs.append(y)
        return torch.cat(outs, 0)

    # ---------------------------------------------------------------- gated delta rule
    def delta(self, layer: int, q, k, v, g, beta):
        H, dk, dv = q.shape[1], q.shape[2], v.shape[2]
        key = (layer, "delta")
        states = [self._get(s, key, (H, dk, dv), torch.float32, q.device) for s in self.batch]
        if self.decode:
            o, new = delta_rule.gated_delta_rule_step(q, k, v, g, beta, torch.stack(states))
            for s, t in zip(self.batch, new):
                s.kv.mixer_state[key] = t
            return o
        outs = []
        for s, st, n, state in zip(self.batch, self.starts, self.lens, states):
            pos = torch.arange(s.kv.length, s.kv.length + n, dtype=torch.int32, device=q.device)
            sl = slice(st, st + n)
            o, new = delta_rule.gated_delta_rule(q[sl], k[sl], v[sl], g[sl], beta[sl], pos,
                                                 initial_state=state if s.kv.length else None, return_state=True)
            s.kv.mixer_state[key] = new
            outs.append(o)
        return torch.cat(outs, 0)


_SUPPORTED = ("Attention", "GatedAttention", "Mamba2Mixer", "GatedDeltaNet")


def needs_hybrid_runner(model) -> bool:
    """True when some layer of ``model`` is not the plain attention + MLP / MoE decoder layer of the fused runner."""
    from ..models.layers import Attention, DecoderLayer

    return any(type(l) is not DecoderLayer or type(l.self_attn) is not Attention for l in model.model.layers)


class HybridRunner(ModelRunner):
    def __init__(self, model, cache, **kw):
        kw.update(use_cuda_graphs=False, shared_prefix_decode=False, tp=None)
        super().__init__(model, cache, **kw)
        for layer in model.model.layers:
            mixers = [m for m in (getattr(layer, "self_attn", None), getattr(layer, "mamba", None)) if m is not None]
            for m in mixers:
                if type(m).__name__ not in _SUPPORTED:
                    raise NotImplementedError(f"the rollout engine has no incremental form of {type(m).__name__} "
                                              f"(model type {model.arch.model_type})")
        if model.arch.hc_mult:
            raise NotImplementedError("the rollout engine does not serve hyper-connection models")

    def _core(self, ids_t, pos_t, slots_t, rows_t, batch, starts):
        from .. import ops
        from ..models.layers import MoE

        lens = [len(s.tokens) for s in batch]
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
        seq = SeqInfo(cu.to(self.device), max(lens), pos_t)
        seq.engine = RecurrentStep(self, batch, starts, slots_t)
        with torch.no_grad():
            h = self.model(ids_t, seq)
        routed = None
        if self.capture_routed:
            tops = [l.mlp.last_topk for l in self.model.model.layers
                    if isinstance(getattr(l, "mlp", None), MoE) and l.mlp.last_topk is not None]
            routed = torch.stack(tops, dim=1) if tops else None
        sel = h[rows_t]
        w = self.model.output_weight
        if sel.is_cuda and sel.dtype == torch.bfloat16:
            logits = ops.gemm(sel.contiguous(), w, out_dtype=torch.float32)
        else:
            logits = sel.float() @ w.float().t()
        return logits, routed
