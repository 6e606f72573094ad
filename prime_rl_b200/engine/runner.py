"""Model runner of the rollout engine: prefill and decode steps over the paged KV cache.

The decoder weights are the same ``CausalLM`` the trainer uses (so trainer and engine share
RoPE / norm / router arithmetic, which keeps the importance ratios near one); this module
only adds the cache writes, the paged attention and the fp32 LM head.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..models import SeqInfo
from ..models.layers import MoE
from ..ops import attention as attn_ops
from .kv_cache import KVCache, SequenceKV


@dataclass
class StepInput:
    """One scheduled sequence: ``tokens`` are the new tokens to run (the whole prompt suffix
    for a prefill, one token for a decode)."""

    kv: SequenceKV
    tokens: list[int]
    want_all_logits: bool = False     # prompt logprobs


class ModelRunner:
    def __init__(self, model, cache: KVCache, fp32_lm_head: bool = True):
        self.model, self.cache, self.arch = model, cache, model.arch
        self.device = next(model.parameters()).device
        self.fp32_lm_head = fp32_lm_head
        self.capture_routed = False
        self.last_routed: torch.Tensor | None = None   # [N, moe_layers, k] of the last step
        self._decode_meta = None                        # (block tables, context lengths) of a pure decode step

    # ------------------------------------------------------------------ attention over pages
    def _attend(self, layer: int, q, k_new, v_new, batch: list[StepInput], starts: list[int], window, sinks):
        """q: [N, Hq, D] for the concatenated new tokens. Context = cached prefix + new tokens."""
        fresh = all(s.kv.length == 0 for s in batch)
        if fresh and sinks is None:
            lens = [len(s.tokens) for s in batch]
            cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
            cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
            return attn_ops.attention(q, k_new, v_new, cu.to(q.device), max(lens), causal=True, window=window)
        if self._decode_meta is not None and sinks is None and window is None:
            from ..ops import paged

            bt, ctx = self._decode_meta
            return paged.paged_decode_raw(q.contiguous(), self.cache.k[layer], self.cache.v[layer], bt, ctx)
        outs = []
        scale = 1.0 / math.sqrt(q.shape[-1])
        rep = q.shape[1] // k_new.shape[1]
        for s, st in zip(batch, starts):
            n = len(s.tokens)
            ctx = s.kv.length + n
            k, v = self.cache.gather(layer, s.kv, ctx)          # includes the tokens just written
            qs = q[st:st + n].float().transpose(0, 1)            # [Hq, n, D]
            ks = k.float().repeat_interleave(rep, dim=1).permute(1, 2, 0)   # [Hq, D, ctx]
            vs = v.float().repeat_interleave(rep, dim=1).transpose(0, 1)    # [Hq, ctx, D]
            sc = (qs @ ks) * scale
            qpos = torch.arange(s.kv.length, ctx, device=q.device)[:, None]
            kpos = torch.arange(ctx, device=q.device)[None, :]
            m = kpos <= qpos
            if window is not None:
                m &= (qpos - kpos) < window
            sc = sc.masked_fill(~m[None], float("-inf"))
            if sinks is not None:
                sk = sinks.float().view(-1, 1, 1).expand(-1, n, 1)
                p = torch.softmax(torch.cat([sc, sk], -1), -1)[..., :-1]
            else:
                p = torch.softmax(sc, -1)
            outs.append((p @ vs).transpose(0, 1).to(q.dtype))
        return torch.cat(outs, 0)

    # ------------------------------------------------------------------ one forward over new tokens
    @torch.no_grad()
    def forward(self, batch: list[StepInput]) -> tuple[torch.Tensor, list[int]]:
        """Runs the new tokens of every sequence, appends their K/V to the cache and returns
        (fp32 logits rows, row offsets): one row per sequence (its last token) unless
        ``want_all_logits`` asks for every position."""
        dev, cache, model = self.device, self.cache, self.model
        ids, pos, slots, starts = [], [], [], []
        for s in batch:
            n = len(s.tokens)
            cache.make_writable_tail(s.kv)
            cache.ensure_capacity(s.kv, s.kv.length + n)
            starts.append(len(ids))
            ids.extend(s.tokens)
            pos.extend(range(s.kv.length, s.kv.length + n))
            slots.extend(cache.slot_mapping(s.kv, s.kv.length, n))
        ids_t = torch.tensor(ids, dtype=torch.long, device=dev)
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slots_t = torch.tensor(slots, dtype=torch.long, device=dev)
        seq = SeqInfo(None, 0, pos_t)
        # a pure decode step on the GPU: one block table / length vector for all layers
        self._decode_meta = None
        if dev.type == "cuda" and all(len(s.tokens) == 1 for s in batch):
            from ..ops import paged

            if paged.available() and self.arch.head_dim == 128:
                max_blocks = max(len(s.kv.pages) for s in batch)
                bt = torch.tensor([s.kv.pages + [0] * (max_blocks - len(s.kv.pages)) for s in batch],
                                  dtype=torch.int32)
                ctx = torch.tensor([s.kv.length + 1 for s in batch], dtype=torch.int32)
                self._decode_meta = (bt.to(dev, non_blocking=True), ctx.to(dev, non_blocking=True))
        h = model.model.embed_tokens(ids_t)
        N = h.shape[0]
        routed = []
        for li, layer in enumerate(model.model.layers):
            at = layer.self_attn
            x = layer.input_layernorm(h)
            qkv = at.qkv_proj(x)
            qd, kd = at.nq * at.D, at.nkv * at.D
            q = qkv[:, :qd].view(N, at.nq, at.D)
            k = qkv[:, qd:qd + kd].view(N, at.nkv, at.D)
            v = qkv[:, qd + kd:].view(N, at.nkv, at.D)
            eps = self.arch.rms_norm_eps
            q = ops.qknorm_rope(q, at.q_norm.weight if at.q_norm is not None else None, pos_t, at.inv_freq, eps)
            k = ops.qknorm_rope(k, at.k_norm.weight if at.k_norm is not None else None, pos_t, at.inv_freq, eps)
            cache.write(li, k, v, slots_t)
            o = self._attend(li, q, k, v.contiguous(), batch, starts, at.window, at.sinks)
            a = at.o_proj(o.reshape(N, qd))
            x2, h = ops.add_rms_norm(a, h, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
            if layer.is_moe:
                m = layer.mlp(x2, seq)
                if self.capture_routed and isinstance(layer.mlp, MoE) and layer.mlp.last_topk is not None:
                    routed.append(layer.mlp.last_topk)
            else:
                m = layer.mlp(x2)
            h = h + m
        for s in batch:
            s.kv.length += len(s.tokens)
        self.last_routed = torch.stack(routed, dim=1) if routed else None
        h = model.model.norm(h)
        rows, offsets = [], []
        for s, st in zip(batch, starts):
            n = len(s.tokens)
            offsets.append(len(rows))
            if s.want_all_logits:
                rows.extend(range(st, st + n))
            else:
                rows.append(st + n - 1)
        sel = h[torch.tensor(rows, dtype=torch.long, device=dev)]
        w = model.output_weight
        if sel.is_cuda and sel.dtype == torch.bfloat16:
            # bf16 operands, fp32 accumulation and fp32 logits (no fp32 copy of the embedding matrix)
            logits = ops.gemm(sel.contiguous(), w, out_dtype=torch.float32)
        else:
            logits = sel.float() @ w.float().t() if self.fp32_lm_head else ops.linear(sel, w).float()
        self._decode_meta = None
        return logits, offsets
