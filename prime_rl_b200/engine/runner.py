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
    # multimodal requests (engine/hybrid.py): rows of ``embeds [n, H]`` replace the token embeddings where
    # ``embed_rows [n]`` is set (image features at the placeholder tokens); ``pos3 [3, n]`` are the tokens' positions
    # on the (time, row, column) axes of the rotary embedding
    embeds: torch.Tensor | None = None
    embed_rows: torch.Tensor | None = None
    pos3: torch.Tensor | None = None


class ModelRunner:
    def __init__(self, model, cache: KVCache, fp32_lm_head: bool = True, use_cuda_graphs: bool = False,
                 max_model_len: int = 8192, tp=None, shared_prefix_decode: bool = False):
        self.model, self.cache, self.arch = model, cache, model.arch
        self.tp = tp                                    # engine/tp.py TPContext: sharded weights, fused reduces
        self.device = next(model.parameters()).device
        self.fp32_lm_head = fp32_lm_head
        self.capture_routed = False
        self.last_routed: torch.Tensor | None = None   # [N, moe_layers, k] of the last step
        self._decode_meta = None                        # (block tables, context lengths, prefix groups) of a decode step
        # samples of one prompt share its pages through the prefix cache: the decode kernels then read those
        # pages once per group of up to 8 sequences instead of once per sequence (csrc/paged_attn.cu)
        self.shared_prefix_decode = shared_prefix_decode and self.device.type == "cuda" and cache.page_size == 16
        self.prefix_splits = 4
        self._group_key = None                          # identity of the batch the current grouping was made for
        self.prefix_stats = {"regroupings": 0, "grouped_sequences": 0, "shared_pages": 0}
        self._cu_batch, self._cu = None, []             # per-sequence cu_seqlens of the current prefix-hit prefill
        # CUDA graphs for decode steps: batch sizes are padded to a multiple of ``graph_bucket``;
        # one page of the cache is reserved as the target of the padding rows
        plain = all(getattr(getattr(l, "self_attn", None), "window", None) is None
                    and getattr(getattr(l, "self_attn", None), "sinks", None) is None for l in model.model.layers)
        self.use_cuda_graphs = use_cuda_graphs and self.device.type == "cuda" and plain
        self.graph_bucket = 8
        self.graph_max_blocks = max(1, (max_model_len + cache.page_size - 1) // cache.page_size)
        self._graphs: dict[int, dict] = {}
        self.scratch_page = cache.blocks.alloc() if self.use_cuda_graphs else 0

    # ------------------------------------------------------------------ attention over pages
    def _attend(self, layer: int, q, k_new, v_new, batch: list[StepInput], starts: list[int], window, sinks):
        """q: [N, Hq, D] for the concatenated new tokens. Context = cached prefix + new tokens."""
        if self._decode_meta is not None and sinks is None and window is None:
            from ..ops import paged

            bt, ctx, prefix = self._decode_meta
            return paged.paged_decode_raw(q.contiguous(), self.cache.k[layer], self.cache.v[layer], bt, ctx,
                                          prefix=prefix)
        fresh = all(s.kv.length == 0 for s in batch)
        if fresh and sinks is None:
            lens = [len(s.tokens) for s in batch]
            cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
            cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
            return attn_ops.attention(q, k_new, v_new, cu.to(q.device), max(lens), causal=True, window=window)
        outs = []
        scale = 1.0 / math.sqrt(q.shape[-1])
        rep = q.shape[1] // k_new.shape[1]
        # prefill on top of a cached prefix (prefix-cache hit, chunked prompt): the tensor-core kernel takes the new
        # tokens as a query slice [prefix, ctx) of the sequence whose K / V are gathered from the pages
        sliced = (q.is_cuda and sinks is None and q.dtype == torch.bfloat16 and q.shape[-1] == 128
                  and attn_ops.default_backend(q.device) == "tcgen05")
        if sliced and self._cu_batch is not batch:
            self._cu_batch = batch
            self._cu = [torch.tensor([0, s.kv.length + len(s.tokens)], dtype=torch.int32).to(q.device, non_blocking=True)
                        for s in batch]
        for bi, (s, st) in enumerate(zip(batch, starts)):
            n = len(s.tokens)
            ctx = s.kv.length + n
            k, v = self.cache.gather(layer, s.kv, ctx)          # includes the tokens just written
            if sliced:
                outs.append(attn_ops.attention(q[st:st + n].contiguous(), k.contiguous(), v.contiguous(), self._cu[bi], ctx,
                                               causal=True, window=window, q_offset=s.kv.length))
                continue
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

    # ------------------------------------------------------------------ decoder over device tensors
    def _core(self, ids_t, pos_t, slots_t, rows_t, batch, starts):
        """ids / positions / cache slots of the N new tokens -> fp32 logits of ``rows_t``. Everything
        here is device work with static shapes for a given N, so a pure decode step can be captured
        in a CUDA graph (``batch`` / ``starts`` are only used by the non-paged attention paths)."""
        model, cache, tp = self.model, self.cache, self.tp
        if batch is not None and any(s.embeds is not None or s.pos3 is not None for s in batch):
            raise NotImplementedError("image inputs are served by the runner of the multimodal families (engine/hybrid.py)")
        seq = SeqInfo(None, 0, pos_t)
        h = model.model.embed_tokens(ids_t)
        N = h.shape[0]
        routed = []
        layers = model.model.layers
        if tp is not None:
            assert tp.calls % 2 == 0, "every forward makes an even number of tensor-parallel reduces"
        add_norm = ops.add_rms_norm if tp is None else tp.reduce
        x = None
        for li, layer in enumerate(layers):
            at = layer.self_attn
            if li == 0:                                 # later layers get their input norm from add_norm below
                x = layer.input_layernorm(h)
            qkv = at.qkv_proj(x)
            eps = self.arch.rms_norm_eps
            # one kernel: split, q / k RMSNorm, rotary, K / V into their cache slots; a paged decode step reads
            # K / V from the cache only, so it asks for no contiguous copies
            paged = self._decode_meta is not None and at.sinks is None and at.window is None
            q, k, v = ops.qkv_rope_to_cache(qkv, at.q_norm.weight if at.q_norm is not None else None,
                                            at.k_norm.weight if at.k_norm is not None else None, pos_t, at.inv_freq,
                                            eps, at.nq, at.nkv, at.D, cache.k[li], cache.v[li], slots_t,
                                            want_kv=not paged)
            o = self._attend(li, q, k, v, batch, starts, at.window, at.sinks)
            a = at.finish(o, x)
            # residual add + norm in one kernel; with TP the same kernel also sums the ranks' partial outputs
            x2, h = add_norm(a, h, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
            if layer.is_moe:
                m = layer.mlp(x2, seq)
                if self.capture_routed and isinstance(layer.mlp, MoE) and layer.mlp.last_topk is not None:
                    routed.append(layer.mlp.last_topk)
            else:
                m = layer.mlp(x2)
            nxt = layers[li + 1].input_layernorm if li + 1 < len(layers) else model.model.norm
            x, h = add_norm(m, h, nxt.weight, nxt.eps)      # the next layer's input norm (or the final norm)
        routed_t = torch.stack(routed, dim=1) if routed else None
        h = x
        sel = h[rows_t]
        w = model.output_weight
        if sel.is_cuda and sel.dtype == torch.bfloat16:
            # bf16 operands, fp32 accumulation and fp32 logits (no fp32 copy of the embedding matrix)
            logits = ops.gemm(sel.contiguous(), w, out_dtype=torch.float32)
        else:
            logits = sel.float() @ w.float().t() if self.fp32_lm_head else ops.linear(sel, w).float()
        return logits, routed_t

    # ------------------------------------------------------------------ CUDA-graph decode
    def _graph_for(self, B: int):
        """Captures one decode step for ``B`` sequences (padded batch size). Static inputs: token
        ids, positions, cache slots, block tables, context lengths; static outputs: logits, routed
        experts. Padding rows point at page 0 / slot 0 of a reserved scratch page."""
        g = self._graphs.get(B)
        if g is not None:
            return g
        dev, ps = self.device, self.cache.page_size
        W = self.graph_max_blocks
        st = {"ids": torch.zeros(B, dtype=torch.long, device=dev), "pos": torch.zeros(B, dtype=torch.int32, device=dev),
              "slots": torch.full((B,), self.scratch_page * ps, dtype=torch.long, device=dev),
              "bt": torch.full((B, W), self.scratch_page, dtype=torch.int32, device=dev),
              "ctx": torch.ones(B, dtype=torch.int32, device=dev), "rows": torch.arange(B, device=dev)}
        st["prefix"] = self._prefix_tensors(B) if self.shared_prefix_decode else None
        self._decode_meta = (st["bt"], st["ctx"], st["prefix"])
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):                      # warm-up: first-use initialisation must not be captured
                self._core(st["ids"], st["pos"], st["slots"], st["rows"], None, None)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits, routed = self._core(st["ids"], st["pos"], st["slots"], st["rows"], None, None)
        st["logits"], st["routed"], st["graph"] = logits, routed, graph
        self._graphs[B] = st
        return st

    # ------------------------------------------------------------------ shared-prefix groups
    def _prefix_tensors(self, B: int):
        """Static device tensors of the group description for a batch of (at most) ``B`` sequences:
        ``page_begin [B]``, ``group_seqs [B / 2, 8]``, ``group_pages [B / 2]`` (all zero / -1 = no groups)."""
        dev = self.device
        n_groups = max(1, B // 2)
        return (torch.zeros(B, dtype=torch.int32, device=dev),
                torch.full((n_groups, 8), -1, dtype=torch.int32, device=dev),
                torch.zeros(n_groups, dtype=torch.int32, device=dev), self.prefix_splits)

    def _update_groups(self, batch, prefix) -> None:
        """Recomputes the grouping when the set of running sequences changed (shared pages are full pages, so a
        grouping stays valid while its members run) and copies it to the device."""
        import numpy as np

        key = (id(prefix[0]),) + tuple(id(s.kv) for s in batch)
        if key == self._group_key:
            return
        self._group_key = key
        from ..ops.paged import group_shared_prefixes

        page_begin_t, group_seqs_t, group_pages_t, _ = prefix
        groups, page_begin = group_shared_prefixes([s.kv.pages for s in batch], [s.kv.length for s in batch],
                                                   self.cache.page_size)
        B, n_slots = page_begin_t.shape[0], group_pages_t.shape[0]
        groups = groups[:n_slots]
        pb = np.zeros(B, dtype=np.int32)
        gs = np.full((n_slots, 8), -1, dtype=np.int32)
        gp = np.zeros(n_slots, dtype=np.int32)
        for gi, (members, shared) in enumerate(groups):
            gs[gi, :len(members)] = members
            gp[gi] = shared
            for i in members:
                pb[i] = shared
        page_begin_t.copy_(torch.from_numpy(pb), non_blocking=False)
        group_seqs_t.copy_(torch.from_numpy(gs), non_blocking=False)
        group_pages_t.copy_(torch.from_numpy(gp), non_blocking=False)
        self.prefix_stats["regroupings"] += 1
        self.prefix_stats["grouped_sequences"] = int((pb > 0).sum())
        self.prefix_stats["shared_pages"] = int(gp.sum())

    def _decode_with_graph(self, batch):
        """Fills the graph's static inputs and replays it. The host side is on the critical path of a decode
        step (the next step cannot start before the sampled tokens were read), so the inputs are assembled in
        one pinned int32 staging array with numpy and cross to the device in ONE copy."""
        import numpy as np

        B = len(batch)
        Bp = (B + self.graph_bucket - 1) // self.graph_bucket * self.graph_bucket
        st = self._graph_for(Bp)
        W, sp, ps = self.graph_max_blocks, self.scratch_page, self.cache.page_size
        stage = st.get("stage")
        if stage is None:
            # [ids | pos | slots | ctx | block table]: int32 [Bp, 4 + W], pinned; a device twin receives the copy
            stage = st["stage"] = torch.empty(Bp, 4 + W, dtype=torch.int32).pin_memory()
            st["stage_np"] = stage.numpy()
            st["stage_dev"] = torch.empty(Bp, 4 + W, dtype=torch.int32, device=self.device)
        arr = st["stage_np"]
        arr[:, 0] = 0
        arr[:, 1] = 0
        arr[:, 2] = sp * ps
        arr[:, 3] = 1
        arr[:, 4:] = sp
        for i, s in enumerate(batch):
            n, pages = s.kv.length, s.kv.pages
            row = arr[i]
            row[0] = s.tokens[0]
            row[1] = n
            row[2] = pages[n // ps] * ps + n % ps
            row[3] = n + 1
            row[4:4 + len(pages)] = pages
        dev = st["stage_dev"]
        dev.copy_(stage, non_blocking=True)
        st["ids"].copy_(dev[:, 0])
        st["pos"].copy_(dev[:, 1])
        st["slots"].copy_(dev[:, 2])
        st["ctx"].copy_(dev[:, 3])
        st["bt"].copy_(dev[:, 4:])
        if st["prefix"] is not None:
            self._update_groups(batch, st["prefix"])
        st["graph"].replay()
        routed = st["routed"][:B].clone() if st["routed"] is not None else None
        return st["logits"][:B].clone(), routed

    # ------------------------------------------------------------------ one forward over new tokens
    @torch.no_grad()
    def forward(self, batch: list[StepInput]) -> tuple[torch.Tensor, list[int]]:
        """Runs the new tokens of every sequence, appends their K/V to the cache and returns
        (fp32 logits rows, row offsets): one row per sequence (its last token) unless
        ``want_all_logits`` asks for every position."""
        dev, cache = self.device, self.cache
        for s in batch:
            cache.make_writable_tail(s.kv)
            cache.ensure_capacity(s.kv, s.kv.length + len(s.tokens))
        decode = dev.type == "cuda" and self.arch.head_dim == 128 and all(len(s.tokens) == 1 for s in batch)
        if decode:
            from ..ops import paged

            decode = paged.available()
        if decode and self.use_cuda_graphs and \
                max(len(s.kv.pages) for s in batch) <= self.graph_max_blocks:
            logits, routed = self._decode_with_graph(batch)
            for s in batch:
                s.kv.length += 1
            self.last_routed = routed
            return logits, list(range(len(batch)))
        ids, pos, slots, starts = [], [], [], []
        for s in batch:
            n = len(s.tokens)
            starts.append(len(ids))
            ids.extend(s.tokens)
            pos.extend(range(s.kv.length, s.kv.length + n))
            slots.extend(cache.slot_mapping(s.kv, s.kv.length, n))
        ids_t = torch.tensor(ids, dtype=torch.long, device=dev)
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slots_t = torch.tensor(slots, dtype=torch.long, device=dev)
        # a pure decode step on the GPU: one block table / length vector for all layers
        self._decode_meta = None
        if decode:
            max_blocks = max(len(s.kv.pages) for s in batch)
            bt = torch.tensor([s.kv.pages + [0] * (max_blocks - len(s.kv.pages)) for s in batch], dtype=torch.int32)
            ctx = torch.tensor([s.kv.length + 1 for s in batch], dtype=torch.int32)
            prefix = None
            if self.shared_prefix_decode and len(batch) > 1:
                if getattr(self, "_eager_prefix", None) is None or self._eager_prefix[0].shape[0] < len(batch):
                    self._eager_prefix = self._prefix_tensors(max(len(batch), 8))
                    self._group_key = None
                self._update_groups(batch, self._eager_prefix)
                prefix = self._eager_prefix
            self._decode_meta = (bt.to(dev, non_blocking=True), ctx.to(dev, non_blocking=True), prefix)
        rows, offsets = [], []
        for s, st in zip(batch, starts):
            n = len(s.tokens)
            offsets.append(len(rows))
            if s.want_all_logits:
                rows.extend(range(st, st + n))
            else:
                rows.append(st + n - 1)
        rows_t = torch.tensor(rows, dtype=torch.long, device=dev)
        logits, routed = self._core(ids_t, pos_t, slots_t, rows_t, batch, starts)
        for s in batch:
            s.kv.length += len(s.tokens)
        self.last_routed = routed
        self._decode_meta = None
        return logits, offsets
