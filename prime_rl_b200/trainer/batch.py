"""Packing of training samples into per-rank micro-batches.

1. every sample is truncated to ``seq_len`` and turned into aligned per-token streams;
2. first-fit-decreasing bin packing into rows of at most ``seq_len`` tokens;
3. rows are balanced over the data-parallel ranks by an attention-aware cost
   (linear + quadratic in the document lengths) with a largest-differencing assignment and
   pairwise swap refinement, so that no rank straggles on long documents;
4. ranks with fewer rows get zero-loss dummy rows: every rank runs the same number of
   micro-steps and collectives stay aligned.

Same contract as the reference's ``prepare_batch``
(src/prime_rl/trainer/batch.py:111-249, :692-913).
"""

from __future__ import annotations

import heapq

from ..transports.batch.types import MicroBatch, TrainingSample


def _cut(x, n):
    return None if x is None else list(x[:n])


def prepare_sample(s: TrainingSample, seq_len: int) -> dict:
    """Aligned per-token streams of one sample, truncated to ``seq_len``."""
    n = min(len(s.token_ids), seq_len)
    k = len(s.token_ids)
    for name in ("mask", "logprobs", "temperatures"):
        if len(getattr(s, name)) != k:
            raise ValueError(f"sample stream '{name}' has {len(getattr(s, name))} entries for {k} tokens")
    adv = s.advantages
    if adv is None:
        live = any(m and (s.rl_weights is None or w != 0) for m, w in zip(s.mask, s.rl_weights or [1.0] * k))
        if live:
            raise ValueError("sample has trainable rl tokens but no advantages")
        adv = [0.0] * k
    d = dict(input_ids=list(s.token_ids[:n]), loss_mask=list(s.mask[:n]), advantages=list(adv[:n]),
             inference_logprobs=list(s.logprobs[:n]), temperatures=list(s.temperatures[:n]), env_name=s.env_name,
             ref_logprobs=_cut(s.ref_logprobs, n), rl_weights=_cut(s.rl_weights, n), ce_weights=_cut(s.ce_weights, n),
             ref_kl_weights=_cut(s.ref_kl_weights, n), routed_experts=s.routed_experts,
             sampling_mask=s.sampling_mask, trace_id=s.trace_id, branch_index=s.branch_index, length=n)
    d["mm_kwargs"], d["mm_token_type_ids"] = s.mm_kwargs, _cut(s.mm_token_type_ids, n)
    if s.mm_kwargs is not None and n < k and s.mm_token_type_ids is not None and any(s.mm_token_type_ids[n:]):
        # the image features of a sample are one tensor for all its images: a cut through (or before) image
        # placeholder tokens would leave features without tokens
        raise ValueError(f"multimodal sample of {k} tokens has image tokens past seq_len={seq_len}; raise seq_len "
                         "or filter such samples")
    return d


def first_fit_decreasing(lengths: list[int], capacity: int) -> list[list[int]]:
    """Indices of the items in each bin."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: list[list[int]] = []
    space: list[int] = []
    for i in order:
        for b in range(len(bins)):
            if lengths[i] <= space[b]:
                bins[b].append(i)
                space[b] -= lengths[i]
                break
        else:
            bins.append([i])
            space.append(capacity - lengths[i])
    return bins


def bin_cost(doc_lengths: list[int], linear: float = 1.0, quadratic: float = 1.0 / 8192) -> float:
    """Relative FLOP estimate of a packed row: matmul work is linear in tokens, causal
    attention quadratic per document."""
    return sum(linear * n + quadratic * n * n for n in doc_lengths)


def balance(costs: list[float], num_ranks: int) -> list[list[int]]:
    """Assign items to ranks with near-equal total cost and equal counts (+-1): largest
    first onto the lightest rank that still has room, then pairwise swaps while they help."""
    n = len(costs)
    per_rank = (n + num_ranks - 1) // num_ranks
    heap = [(0.0, r) for r in range(num_ranks)]
    out: list[list[int]] = [[] for _ in range(num_ranks)]
    for i in sorted(range(n), key=lambda i: -costs[i]):
        popped = []
        while True:
            load, r = heapq.heappop(heap)
            if len(out[r]) < per_rank:
                break
            popped.append((load, r))
        out[r].append(i)
        heapq.heappush(heap, (load + costs[i], r))
        for p in popped:
            heapq.heappush(heap, p)
    loads = [sum(costs[i] for i in items) for items in out]
    improved = True
    while improved:
        improved = False
        hi, lo = max(range(num_ranks), key=loads.__getitem__), min(range(num_ranks), key=loads.__getitem__)
        gap = loads[hi] - loads[lo]
        best = None
        for a in out[hi]:
            for b in out[lo]:
                delta = costs[a] - costs[b]
                if 0 < delta < gap and (best is None or abs(gap - 2 * delta) < best[0]):
                    best = (abs(gap - 2 * delta), a, b, delta)
        if best is not None and best[0] < gap - 1e-9:
            _, a, b, delta = best
            out[hi].remove(a); out[lo].remove(b)
            out[hi].append(b); out[lo].append(a)
            loads[hi] -= delta; loads[lo] += delta
            improved = True
    return out


def _merge_optional(rows: list[dict], key: str, default: float) -> list[float] | None:
    if all(r[key] is None for r in rows):
        return None
    out: list[float] = []
    for r in rows:
        if r[key] is not None:
            out.extend(r[key])
        elif key == "rl_weights":
            out.extend([1.0] * r["length"])       # absent rl stream = weight 1 on the loss mask
        else:
            out.extend([default] * r["length"])
    return out


def _pack_row(rows: list[dict], pad_to: int) -> MicroBatch:
    import numpy as np

    ids, mask, adv, lps, temps, pos, envs, lens = [], [], [], [], [], [], [], []
    for r in rows:
        n = r["length"]
        ids.extend(r["input_ids"]); mask.extend(r["loss_mask"]); adv.extend(r["advantages"])
        lps.extend(r["inference_logprobs"]); temps.extend(r["temperatures"]); pos.extend(range(n))
        envs.append(r["env_name"]); lens.append(n)
    mb = MicroBatch(input_ids=ids, loss_mask=mask, advantages=adv, inference_logprobs=lps, position_ids=pos,
                    sequence_lengths=lens, temperatures=temps, env_names=envs, seq_lens=list(lens),
                    ref_logprobs=_merge_optional(rows, "ref_logprobs", 0.0),
                    rl_weights=_merge_optional(rows, "rl_weights", 1.0),
                    ce_weights=_merge_optional(rows, "ce_weights", 0.0),
                    ref_kl_weights=_merge_optional(rows, "ref_kl_weights", 0.0))
    if any(r["trace_id"] is not None for r in rows):
        mb.trace_ids = [r["trace_id"] or "" for r in rows]
        mb.branch_indices = [r["branch_index"] if r["branch_index"] is not None else -1 for r in rows]
    if all(r["routed_experts"] is not None for r in rows):
        from ..transports.batch.types import RoutedExperts

        arrs = [np.frombuffer(r["routed_experts"].data, dtype=np.dtype(r["routed_experts"].dtype))
                .reshape(r["routed_experts"].shape)[: r["length"]] for r in rows]
        full = np.concatenate(arrs, 0)
        mb.routed_experts = RoutedExperts(data=full.tobytes(), shape=list(full.shape), dtype=str(full.dtype))
    if any(r["sampling_mask"] is not None for r in rows):
        from ..transports.batch.types import SamplingMask

        counts, idbufs = [], []
        for r in rows:
            sm = r["sampling_mask"]
            if sm is None:
                counts.append(np.zeros(r["length"], np.int32))
            else:
                c = np.frombuffer(sm.counts, np.int32)[: r["length"]]
                counts.append(c)
                idbufs.append(np.frombuffer(sm.ids, np.int32)[: int(c.sum())])
        mb.sampling_mask = SamplingMask(ids=(np.concatenate(idbufs) if idbufs else np.zeros(0, np.int32)).tobytes(),
                                        counts=np.concatenate(counts).tobytes())
    if any(r.get("mm_kwargs") is not None for r in rows):
        from ..transports.batch.types import EncodedTensor

        # image tensors of the row's samples, concatenated along dim 0 in token order
        keys = sorted({k for r in rows if r.get("mm_kwargs") for k in r["mm_kwargs"]})
        merged = {}
        for key in keys:
            parts = [r["mm_kwargs"][key] for r in rows if r.get("mm_kwargs") and key in r["mm_kwargs"]]
            arrs = [np.frombuffer(e.data, dtype=np.dtype(e.dtype)).reshape(e.shape) for e in parts]
            full = np.concatenate(arrs, 0)
            merged[key] = EncodedTensor(dtype=str(full.dtype), shape=list(full.shape), data=full.tobytes())
        mb.mm_kwargs = merged
        types: list[int] = []
        for r in rows:
            types.extend(r.get("mm_token_type_ids") or [0] * r["length"])
        mb.mm_token_type_ids = types
    total = len(ids)
    if pad_to > 1 and total % pad_to:
        _pad(mb, pad_to - total % pad_to)
    return mb


def _pad(mb: MicroBatch, n: int) -> None:
    """Appends a loss-free padding document of ``n`` tokens."""
    mb.input_ids.extend([0] * n); mb.loss_mask.extend([False] * n); mb.advantages.extend([0.0] * n)
    mb.inference_logprobs.extend([0.0] * n); mb.temperatures.extend([1.0] * n); mb.position_ids.extend(range(n))
    mb.sequence_lengths.append(n); mb.seq_lens.append(n); mb.env_names.append("")
    for name, fill in (("ref_logprobs", 0.0), ("rl_weights", 0.0), ("ce_weights", 0.0), ("ref_kl_weights", 0.0)):
        v = getattr(mb, name)
        if v is not None:
            v.extend([fill] * n)
    if mb.trace_ids is not None:
        mb.trace_ids.append(""); mb.branch_indices.append(-1)
    if mb.mm_token_type_ids is not None:
        mb.mm_token_type_ids.extend([0] * n)


def dummy_micro_batch(like: MicroBatch, length: int | None = None) -> MicroBatch:
    """Zero-loss row (same optional streams as ``like``) so that every rank runs the same
    number of micro-steps."""
    n = length or min(len(like.input_ids), 16) or 16
    z = lambda v: [0.0] * n if v is not None else None  # noqa: E731
    return MicroBatch(input_ids=[0] * n, loss_mask=[False] * n, advantages=[0.0] * n, inference_logprobs=[0.0] * n,
                      position_ids=list(range(n)), sequence_lengths=[n], temperatures=[1.0] * n, env_names=[""],
                      seq_lens=[n], ref_logprobs=z(like.ref_logprobs), rl_weights=z(like.rl_weights),
                      ce_weights=z(like.ce_weights), ref_kl_weights=z(like.ref_kl_weights),
                      trace_ids=[""] if like.trace_ids is not None else None,
                      branch_indices=[-1] if like.branch_indices is not None else None)


def prepare_batch(samples: list[TrainingSample], *, seq_len: int, num_train_workers: int,
                  pad_to_multiple_of: int = 1) -> list[list[MicroBatch]]:
    """-> grid[dp_rank][micro_step]"""
    rows = [prepare_sample(s, seq_len) for s in samples]
    if not rows:
        raise ValueError("cannot pack an empty batch")
    bins = first_fit_decreasing([r["length"] for r in rows], seq_len)
    packed = [_pack_row([rows[i] for i in b], pad_to_multiple_of) for b in bins]
    for mb in packed:   # alignment check: every stream is as long as the row
        n = len(mb.input_ids)
        for name in ("loss_mask", "advantages", "inference_logprobs", "position_ids", "temperatures"):
            assert len(getattr(mb, name)) == n, f"stream {name} misaligned after packing"
        assert sum(mb.sequence_lengths) == n
    costs = [bin_cost(mb.sequence_lengths) for mb in packed]
    assign = balance(costs, num_train_workers)
    steps = max(len(a) for a in assign)
    grid = []
    for a in assign:
        mbs = [packed[i] for i in a]
        while len(mbs) < steps:
            mbs.append(dummy_micro_batch(packed[0]))
        grid.append(mbs)
    return grid
