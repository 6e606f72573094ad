"""Front end of the paged-attention decode kernel (``csrc/paged_attn.cu``)."""

from __future__ import annotations

import math

import torch

from .. import native
from . import _runtime as rt


def available() -> bool:
    try:
        return hasattr(native.cuda(), "prb_paged_decode")
    except Exception:
        return False


def paged_decode_ref(q, kpool, vpool, block_tables, ctx_lens, scale=None):
    """fp32 reference: q [B, Hq, D]; pools [pages, page_size, Hkv, D]."""
    B, Hq, D = q.shape
    ps, Hkv = kpool.shape[1], kpool.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    for b in range(B):
        n = int(ctx_lens[b])
        pages = block_tables[b, : (n + ps - 1) // ps].long()
        k = kpool[pages].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, 1)
        v = vpool[pages].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * scale
        out[b] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).to(q.dtype)
    return out


def group_shared_prefixes(page_lists: list[list[int]], lengths: list[int], page_size: int = 16,
                          min_pages: int = 4, max_group: int = 8):
    """Finds sequences whose leading pages are the same physical pages (samples of one prompt served from the
    prefix cache). Returns ``(groups, page_begin)``: ``groups`` = list of (member indices (<= 8), shared page
    count), ``page_begin[i]`` = pages of sequence i that a group covers (0 when it is in no group). Only pages
    that are completely filled for every member count: those are never written again, so a grouping stays
    valid for as long as its members run."""
    by_first: dict[int, list[int]] = {}
    for i, pages in enumerate(page_lists):
        if pages:
            by_first.setdefault(pages[0], []).append(i)
    groups, page_begin = [], [0] * len(page_lists)
    for members in by_first.values():
        if len(members) < 2:
            continue
        for c in range(0, len(members), max_group):
            chunk = members[c:c + max_group]
            if len(chunk) < 2:
                continue
            lead = page_lists[chunk[0]]
            shared = min(min(lengths[i] for i in chunk) // page_size, *(len(page_lists[i]) for i in chunk))
            for i in chunk[1:]:
                other = page_lists[i]
                n = 0
                while n < shared and other[n] == lead[n]:
                    n += 1
                shared = n
            if shared >= min_pages:
                groups.append((chunk, shared))
                for i in chunk:
                    page_begin[i] = shared
    return groups, page_begin


def paged_decode_raw(q, kpool, vpool, block_tables, ctx_lens, scale=None, splits: int | None = None, prefix=None):
    """``prefix = (page_begin [B], group_seqs [groups, 8], group_pages [groups], prefix_splits)`` (int32 device
    tensors): shared leading pages are read once per group by the group kernel, see ``group_shared_prefixes``."""
    B, Hq, D = q.shape
    ps, Hkv = kpool.shape[1], kpool.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if splits is None:
        ctas = B * Hkv
        splits = 1 if ctas >= 256 else min(16, max(1, 296 // max(ctas, 1)))
    if prefix is not None:
        page_begin, group_seqs, group_pages, psplits = prefix
        total = splits + psplits
        out = torch.empty_like(q)
        o_part = torch.empty(B, Hq, total, D, dtype=torch.float32, device=q.device)
        ml_part = torch.empty(B, Hq, total, 2, dtype=torch.float32, device=q.device)
        rc = rt.lib().prb_paged_decode_prefix(q.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), block_tables.data_ptr(),
                                              ctx_lens.data_ptr(), out.data_ptr(), o_part.data_ptr(), ml_part.data_ptr(),
                                              B, Hq, Hkv, D, ps, block_tables.shape[1], splits, float(scale),
                                              page_begin.data_ptr(), group_seqs.data_ptr(), group_pages.data_ptr(),
                                              group_seqs.shape[0], int(psplits), rt.stream_ptr(q.device))
        rt.check(rc, "prb_paged_decode_prefix")
        return out
    out = torch.empty_like(q)
    o_part = ml_part = None
    if splits > 1:
        o_part = torch.empty(B, Hq, splits, D, dtype=torch.float32, device=q.device)
        ml_part = torch.empty(B, Hq, splits, 2, dtype=torch.float32, device=q.device)
    rc = rt.lib().prb_paged_decode(q.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), block_tables.data_ptr(),
                                   ctx_lens.data_ptr(), out.data_ptr(), rt.ptr(o_part), rt.ptr(ml_part), B, Hq, Hkv, D,
                                   ps, block_tables.shape[1], splits, float(scale), rt.stream_ptr(q.device))
    rt.check(rc, "prb_paged_decode")
    return out


def paged_decode(q, cache, layer: int, batch) -> torch.Tensor:
    """q: [B, Hq, D] (one new token per sequence, K/V already written); ``batch`` gives the
    sequences' page lists and lengths (engine/runner.py StepInput)."""
    B = len(batch)
    max_blocks = max(len(s.kv.pages) for s in batch)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    for i, s in enumerate(batch):
        bt[i, : len(s.kv.pages)] = torch.tensor(s.kv.pages, dtype=torch.int32)
    ctx = torch.tensor([s.kv.length + 1 for s in batch], dtype=torch.int32)
    dev = q.device
    return paged_decode_raw(q.contiguous(), cache.k[layer], cache.v[layer], bt.to(dev, non_blocking=True),
                            ctx.to(dev, non_blocking=True))
