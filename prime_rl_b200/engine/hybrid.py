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

The states live in one pool per layer (``StatePool``: ``[slots, ...]``); a sequence owns one slot from its first step
until its ``SequenceKV`` object dies (request finished, or preempted: a preempted request recomputes from its tokens).
A decode step advances the slots of all running sequences in place with one launch per layer
(``csrc/recurrent_step.cu``). A recurrent state cannot be shared
through the page-level prefix cache, so engines of these families run without it.

The reference serves these families through vLLM's hybrid KV-cache manager (one Mamba state slot per request next to
the attention pages); its own code only configures it (packages/prime-rl-configs/src/prime_rl/configs/inference.py).
"""

from __future__ import annotations

import torch

from ..models.layers import SeqInfo
from ..ops import delta_rule, ssm
from .runner import ModelRunner, StepInput


class StatePool:
    """Per (layer, kind) one tensor ``[capacity, ...]``; every live sequence owns one row index (its slot) in all of
    them. Slots are handed out at a sequence's first step and return when its ``SequenceKV`` object dies."""

    def __init__(self, device):
        self.device, self.capacity = device, 0
        self.tensors: dict[tuple, torch.Tensor] = {}
        self.free: list[int] = []
        self.next = 0

    def slot(self, kv) -> int:
        import weakref

        sl = getattr(kv, "state_slot", None)
        if sl is None:
            sl = self.free.pop() if self.free else self.next
            if sl == self.next:
                self.next += 1
            kv.state_slot = sl
            weakref.finalize(kv, self.free.append, sl)
        return sl

    def get(self, key, shape, dtype) -> torch.Tensor:
        t = self.tensors.get(key)
        need = max(self.next, 1)
        if t is None or t.shape[0] < need:
            cap = max(8, 2 * need)
            new = torch.zeros((cap, *shape), dtype=dtype, device=self.device)
            if t is not None:
                new[: t.shape[0]] = t
            self.tensors[key] = t = new
        return t

    def clear(self, slot: int) -> None:
        for t in self.tensors.values():
            if slot < t.shape[0]:
                t[slot].zero_()

    def copy(self, src: int, dst: int) -> None:
        """State of slot ``src`` into slot ``dst`` in every pool (a sequence forked from another one)."""
        for key, t in list(self.tensors.items()):
            if t.shape[0] <= max(src, dst):
                t = self.get(key, tuple(t.shape[1:]), t.dtype)
            t[dst].copy_(t[src])


class RecurrentStep:
    def __init__(self, runner: "HybridRunner", batch: list[StepInput], starts: list[int], slots_t: torch.Tensor):
        self.runner, self.batch, self.starts, self.slots = runner, batch, starts, slots_t
        self.pool = runner.pool
        self.lens = [len(s.tokens) for s in batch]
        self.decode = all(n == 1 and s.kv.length > 0 for n, s in zip(self.lens, batch))
        self.state_slots = [self.pool.slot(s.kv) for s in batch]
        for s, sl in zip(batch, self.state_slots):
            if s.kv.length == 0:
                self.pool.clear(sl)                 # a fresh (or restarted) sequence starts from nothing
        self._slots_t = None

    @property
    def slots_t(self) -> torch.Tensor:
        if self._slots_t is None:
            self._slots_t = torch.tensor(self.state_slots, dtype=torch.int32, device=self.pool.device)
        return self._slots_t

    # ---------------------------------------------------------------- attention
    def attend(self, layer: int, q, k, v, window, sinks):
        cache = self.runner.cache
        Hkv, D = k.shape[1], k.shape[2]
        cache.k[layer].view(-1, Hkv, D).index_copy_(0, self.slots, k.to(cache.k.dtype))
        cache.v[layer].view(-1, Hkv, D).index_copy_(0, self.slots, v.to(cache.v.dtype))
        return self.runner._attend(layer, q, k, v, self.batch, self.starts, window, sinks)

    # ---------------------------------------------------------------- per-sequence stores (model-specific mixers)
    def sequences(self):
        """(slice of the new tokens in the packed step, the sequence's store, tokens before them) per sequence."""
        for s, st, n in zip(self.batch, self.starts, self.lens):
            yield slice(st, st + n), s.kv.__dict__.setdefault("latent", {}), s.kv.length

    @staticmethod
    def append(store: dict, key, rows: torch.Tensor, length: int) -> torch.Tensor:
        """Growing buffer ``store[key]`` (capacity doubles): rows ``[length, length + n)`` are written; returns the
        filled part."""
        buf = store.get(key)
        need = length + rows.shape[0]
        if buf is None or buf.shape[0] < need:
            new = torch.empty((max(64, 2 * need), rows.shape[1]), dtype=rows.dtype, device=rows.device)
            if buf is not None and length:
                new[:length] = buf[:length]
            store[key] = buf = new
        buf[length:need] = rows
        return buf[:need]

    def sparse_mla(self, layer: int, index_source: int, sq, skv, idx_in, topk: int, scale: float, d_v: int):
        """Multi-head latent attention over the keys the indexer selects: every sequence keeps the latent K / V row
        and the indexer key of each of its tokens per layer; layers that share a selection read the one their
        source layer made in this step."""
        from ..ops import sparse_mla as sm

        outs = []
        for s, st, n in zip(self.batch, self.starts, self.lens):
            r = slice(st, st + n)
            L = s.kv.length
            store = s.kv.__dict__.setdefault("latent", {})
            kv_all = self.append(store, (layer, "skv"), skv[r], L)
            picked = s.kv.__dict__.setdefault("dsa_indices", {})
            if idx_in is not None:
                q_i, k_i, w_i = idx_in
                k_all = self.append(store, (layer, "idx_k"), k_i[r], L)
                ke = torch.arange(L + 1, L + n + 1, dtype=torch.int32, device=sq.device)
                picked[layer] = sm.dsa_indexer_topk(q_i[r], k_all, w_i[r], torch.zeros_like(ke), ke, topk)
            indices = picked[index_source]
            outs.append(sm.sparse_mla_attention(sq[r].contiguous(), kv_all, indices, scale, d_v))
        return torch.cat(outs, 0)

    # ---------------------------------------------------------------- convolution
    def conv(self, layer: int, x, weight, bias, activation="silu"):
        K, C = weight.shape[1], x.shape[1]
        tails = self.pool.get((layer, "conv"), (K - 1, C), x.dtype)
        if self.decode:
            idx = self.slots_t.long()
            y, new = ssm.conv1d_step(tails[idx], x, weight, bias, activation)
            tails.index_copy_(0, idx, new)
            return y
        outs = []
        for sl, st, n in zip(self.state_slots, self.starts, self.lens):
            y, new = ssm.conv1d_window(tails[sl], x[st:st + n], weight, bias, activation)
            tails[sl] = new
            outs.append(y)
        return torch.cat(outs, 0)

    # ---------------------------------------------------------------- Mamba-2
    def mamba(self, layer: int, x, dt, A, B, C, D, chunk: int):
        H, P, N = x.shape[1], x.shape[2], B.shape[2]
        states = self.pool.get((layer, "ssm"), (H, P, N), torch.float32)
        if self.decode:
            if x.is_cuda and N % 4 == 0:
                from ..ops import _runtime as rt

                n, G = x.shape[0], B.shape[1]
                xf, dtf = x.float().contiguous(), dt.float().contiguous()
                Bf, Cf = B.float().contiguous(), C.float().contiguous()
                Af, Df = A.float().contiguous(), (D.float().contiguous() if D is not None else None)
                y = torch.empty(n, H, P, dtype=torch.float32, device=x.device)
                rt.check(rt.lib().prb_mamba2_step(states.data_ptr(), self.slots_t.data_ptr(), xf.data_ptr(), dtf.data_ptr(),
                                                  Af.data_ptr(), Bf.data_ptr(), Cf.data_ptr(), rt.ptr(Df), y.data_ptr(), n,
                                                  H, P, N, G, rt.stream_ptr(x.device)), "prb_mamba2_step")
                return y
            idx = self.slots_t.long()
            y, new = ssm.mamba2_step(x, dt, A, B, C, D, states[idx])
            states.index_copy_(0, idx, new)
            return y
        outs = []
        for s, sl, st, n in zip(self.batch, self.state_slots, self.starts, self.lens):
            pos = torch.arange(s.kv.length, s.kv.length + n, dtype=torch.int32, device=x.device)
            r = slice(st, st + n)
            y, new = ssm.mamba2_scan(x[r], dt[r], A, B[r], C[r], D, pos, chunk=chunk,
                                     initial_state=states[sl] if s.kv.length else None, return_state=True)
            states[sl] = new
            outs.append(y)
        return torch.cat(outs, 0)

    # ---------------------------------------------------------------- gated delta rule
    def delta(self, layer: int, q, k, v, g, beta):
        H, dk, dv = q.shape[1], q.shape[2], v.shape[2]
        states = self.pool.get((layer, "delta"), (H, dk, dv), torch.float32)
        if self.decode:
            if q.is_cuda and dv <= 1024:
                from ..ops import _runtime as rt

                n = q.shape[0]
                qf = (delta_rule._l2norm(q.float()) * dk ** -0.5).contiguous()
                kf = delta_rule._l2norm(k.float()).contiguous()
                vf, gf, bf = v.float().contiguous(), g.float().contiguous(), beta.float().contiguous()
                o = torch.empty(n, H, dv, dtype=torch.float32, device=q.device)
                rt.check(rt.lib().prb_delta_rule_step(states.data_ptr(), self.slots_t.data_ptr(), qf.data_ptr(),
                                                      kf.data_ptr(), vf.data_ptr(), gf.data_ptr(), bf.data_ptr(),
                                                      o.data_ptr(), n, H, dk, dv, rt.stream_ptr(q.device)),
                         "prb_delta_rule_step")
                return o
            idx = self.slots_t.long()
            o, new = delta_rule.gated_delta_rule_step(q, k, v, g, beta, states[idx])
            states.index_copy_(0, idx, new)
            return o
        outs = []
        for s, sl, st, n in zip(self.batch, self.state_slots, self.starts, self.lens):
            pos = torch.arange(s.kv.length, s.kv.length + n, dtype=torch.int32, device=q.device)
            r = slice(st, st + n)
            o, new = delta_rule.gated_delta_rule(q[r], k[r], v[r], g[r], beta[r], pos,
                                                 initial_state=states[sl] if s.kv.length else None, return_state=True)
            states[sl] = new
            outs.append(o)
        return torch.cat(outs, 0)


_SUPPORTED = ("Attention", "GatedAttention", "Mamba2Mixer", "GatedDeltaNet", "SparseMLAAttention", "DSV4Attention")


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
        self.pool = StatePool(self.device)
        self.mrope_section = (11, 11, 10)           # set by the engine when it serves image inputs

    def fork_state(self, src_kv, dst_kv) -> None:
        """Everything this runner keeps for ``src_kv`` besides the pages (recurrent states, convolution tails, latent
        rows, pending compressor projections) copied for ``dst_kv``: a second sample of the same prompt continues from
        the first one's prefill instead of running the prompt again."""
        import copy

        if getattr(src_kv, "state_slot", None) is not None:
            self.pool.copy(src_kv.state_slot, self.pool.slot(dst_kv))

        def clone(v):
            if torch.is_tensor(v):
                return v.clone()
            if isinstance(v, dict):
                return {k: clone(x) for k, x in v.items()}
            return copy.copy(v)

        latent = src_kv.__dict__.get("latent")
        if latent is not None:
            dst_kv.latent = clone(latent)

    def _core(self, ids_t, pos_t, slots_t, rows_t, batch, starts):
        from .. import ops
        from ..models.layers import MoE

        lens = [len(s.tokens) for s in batch]
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
        seq = SeqInfo(cu.to(self.device), max(lens), pos_t)
        seq.engine = RecurrentStep(self, batch, starts, slots_t)
        embeds = None
        if any(s.embeds is not None or s.pos3 is not None for s in batch):
            # image features in place of the placeholder embeddings; positions on three axes (text tokens: the same
            # value on all of them)
            from ..models.vision import mrope_angles

            embeds = self.model.model.embed_tokens(ids_t)
            pos3 = pos_t.to(torch.long).unsqueeze(0).repeat(3, 1)
            for s, st, n in zip(batch, starts, lens):
                if s.embeds is not None:
                    rows = s.embed_rows.to(self.device)
                    embeds[st:st + n][rows] = s.embeds.to(self.device, embeds.dtype)[rows]
                if s.pos3 is not None:
                    pos3[:, st:st + n] = s.pos3.to(self.device)
            arch = self.model.arch
            rd = arch.rotary_dim
            inv_freq = 1.0 / (arch.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float32, device=self.device) / rd))
            seq.mrope_angles = mrope_angles(pos3, inv_freq, self.mrope_section)
        with torch.no_grad():
            h = self.model(ids_t, seq, inputs_embeds=embeds)
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
