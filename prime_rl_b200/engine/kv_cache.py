"""Paged KV cache: fixed-size pages (16 tokens by default) in one preallocated bf16 pool per
layer, block tables per sequence, reference-counted pages so that the samples of one prompt
share its prefix pages (copy-on-write on the last, partially filled page).

Takes the place of vLLM's block manager in the reference's inference stack
(src/prime_rl/inference/vllm/*); `cache_salt` from the request keys the prefix cache so
that KV computed under an older policy version is never reused.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


class OutOfPages(RuntimeError):
    pass


class BlockManager:
    """Page allocator with reference counts and a hash-keyed prefix cache."""

    def __init__(self, num_pages: int, page_size: int):
        self.num_pages, self.page_size = num_pages, page_size
        self.free = list(range(num_pages - 1, -1, -1))
        self.refcount = [0] * num_pages
        self.prefix_cache: dict[tuple, int] = {}     # (salt, tokens-so-far hash) -> page id
        self.page_key: dict[int, tuple] = {}
        self.evictable = 0                            # cached pages that no sequence holds any more

    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def num_available(self) -> int:
        """Pages an allocation can get: the free list plus cached prefix pages nobody is using."""
        return len(self.free) + self.evictable

    @property
    def usage(self) -> float:
        return 1.0 - self.num_available / max(1, self.num_pages)

    def alloc(self) -> int:
        if not self.free:
            self._evict_cached()
        if not self.free:
            raise OutOfPages()
        p = self.free.pop()
        self.refcount[p] = 1
        return p

    def _evict_cached(self) -> None:
        """Pages held only by the prefix cache can be reclaimed."""
        for key, p in list(self.prefix_cache.items()):
            if self.refcount[p] == 1:
                del self.prefix_cache[key]
                self.page_key.pop(p, None)
                self.refcount[p] = 0
                self.evictable -= 1
                self.free.append(p)
                if len(self.free) >= 8:
                    break

    def incref(self, p: int) -> None:
        if self.refcount[p] == 1 and p in self.page_key:
            self.evictable -= 1                      # a sequence picks a cached page up again
        self.refcount[p] += 1

    def release(self, pages: list[int]) -> None:
        for p in pages:
            self.refcount[p] -= 1
            if self.refcount[p] == 0:
                key = self.page_key.pop(p, None)
                if key is not None:
                    self.prefix_cache.pop(key, None)
                self.free.append(p)
            elif self.refcount[p] == 1 and p in self.page_key:
                self.evictable += 1                  # only the cache holds it now

    # prefix cache -----------------------------------------------------------------
    def lookup_prefix(self, salt: str, tokens: list[int]) -> list[int]:
        """Longest run of full pages of ``tokens`` already cached under ``salt``."""
        pages, h = [], hash(salt)
        ps = self.page_size
        for i in range(0, len(tokens) - len(tokens) % ps, ps):
            h = hash((h, tuple(tokens[i:i + ps])))
            p = self.prefix_cache.get((salt, h))
            if p is None:
                break
            pages.append(p)
        for p in pages:
            self.incref(p)
        return pages

    def register_prefix(self, salt: str, tokens: list[int], pages: list[int]) -> None:
        h = hash(salt)
        ps = self.page_size
        for n, i in enumerate(range(0, len(tokens) - len(tokens) % ps, ps)):
            h = hash((h, tuple(tokens[i:i + ps])))
            key = (salt, h)
            if key not in self.prefix_cache and n < len(pages) and pages[n] not in self.page_key:
                self.prefix_cache[key] = pages[n]
                self.refcount[pages[n]] += 1      # the cache holds one reference
                self.page_key[pages[n]] = key

    def clear_prefix_cache(self) -> None:
        for key, p in list(self.prefix_cache.items()):
            self.refcount[p] -= 1
            if self.refcount[p] == 0:
                self.free.append(p)
        self.prefix_cache.clear()
        self.page_key.clear()
        self.evictable = 0


@dataclass
class SequenceKV:
    pages: list[int] = field(default_factory=list)
    length: int = 0            # tokens whose K/V are in the cache


@dataclass
class HostKV:
    """K / V of one preempted sequence in host memory: ``data`` [2, layers, pages, page_size, kv_heads, head_dim]."""
    data: torch.Tensor
    length: int
    ready: object = None

    @property
    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def to_file(self, path) -> dict:
        """Writes the K / V bytes to ``path`` (a file in shared memory when the peer engine runs on the same box) and
        returns the description the importing side needs (``from_file``)."""
        if self.ready is not None:
            self.ready.synchronize()
        self.data.contiguous().view(torch.uint8).numpy().tofile(str(path))
        return {"path": str(path), "shape": list(self.data.shape), "dtype": str(self.data.dtype).replace("torch.", ""),
                "length": int(self.length)}

    @classmethod
    def from_file(cls, meta: dict, delete: bool = True) -> "HostKV":
        import os

        dtype = getattr(torch, meta["dtype"])
        shape = tuple(int(x) for x in meta["shape"])
        n = 1
        for d in shape:
            n *= d
        raw = torch.from_file(str(meta["path"]), shared=False, size=n * torch.empty((), dtype=dtype).element_size(),
                              dtype=torch.uint8)
        data = raw.view(dtype).view(shape).clone()
        if delete:
            try:
                os.unlink(meta["path"])
            except OSError:
                pass
        return cls(data, int(meta["length"]), None)


class KVCache:
    """Pools ``k[layer]``, ``v[layer]``: ``[num_pages, page_size, kv_heads, head_dim]``."""

    def __init__(self, num_layers: int, num_pages: int, page_size: int, kv_heads: int, head_dim: int, dtype, device):
        self.page_size = page_size
        self.k = torch.zeros(num_layers, num_pages, page_size, kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.blocks = BlockManager(num_pages, page_size)

    def ensure_capacity(self, seq: SequenceKV, new_len: int) -> None:
        need = (new_len + self.page_size - 1) // self.page_size
        while len(seq.pages) < need:
            seq.pages.append(self.blocks.alloc())

    def make_writable_tail(self, seq: SequenceKV) -> None:
        """Copy-on-write: a shared last page is duplicated before this sequence appends to it."""
        if not seq.pages or seq.length % self.page_size == 0:
            return
        tail = seq.pages[-1]
        if self.blocks.refcount[tail] > 1:
            new = self.blocks.alloc()
            self.k[:, new].copy_(self.k[:, tail])
            self.v[:, new].copy_(self.v[:, tail])
            self.blocks.release([tail])
            seq.pages[-1] = new

    def fork(self, seq: SequenceKV) -> SequenceKV:
        for p in seq.pages:
            self.blocks.incref(p)
        return SequenceKV(list(seq.pages), seq.length)

    def free(self, seq: SequenceKV) -> None:
        self.blocks.release(seq.pages)
        seq.pages, seq.length = [], 0

    # host offload ---------------------------------------------------------------------
    def swap_out(self, seq: SequenceKV, pin: bool = True) -> "HostKV":
        """Copies the sequence's pages (all layers, K and V) to host memory and gives the pages back. The copy is
        issued on the current stream into pinned memory; ``HostKV.ready`` fires when it has landed."""
        n = len(seq.pages)
        idx = torch.tensor(seq.pages, dtype=torch.long, device=self.k.device)
        shape = (2, self.k.shape[0], n, *self.k.shape[2:])
        host = torch.empty(shape, dtype=self.k.dtype, device="cpu")
        if pin and self.k.is_cuda:
            host = host.pin_memory()
        host[0].copy_(self.k.index_select(1, idx), non_blocking=True)
        host[1].copy_(self.v.index_select(1, idx), non_blocking=True)
        ready = None
        if self.k.is_cuda:
            ready = torch.cuda.Event()
            ready.record()
        out = HostKV(host, seq.length, ready)
        self.free(seq)
        return out

    def swap_in(self, seq: SequenceKV, host: "HostKV") -> None:
        """Fresh pages for ``seq`` filled from ``host`` (raises ``OutOfPages`` before touching anything when
        there are not enough)."""
        n = host.data.shape[2]
        if self.blocks.num_available < n:
            raise OutOfPages()
        pages = [self.blocks.alloc() for _ in range(n)]
        idx = torch.tensor(pages, dtype=torch.long, device=self.k.device)
        if host.ready is not None:
            host.ready.synchronize()
        dev = host.data.to(self.k.device, non_blocking=True)
        self.k.index_copy_(1, idx, dev[0])
        self.v.index_copy_(1, idx, dev[1])
        seq.pages, seq.length = pages, host.length

    def slot_mapping(self, seq: SequenceKV, start: int, n: int) -> list[int]:
        """Flat slot (page * page_size + offset) of tokens [start, start + n)."""
        ps = self.page_size
        return [seq.pages[t // ps] * ps + t % ps for t in range(start, start + n)]

    def write(self, layer: int, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
        """k, v: [n, kv_heads, head_dim]; slots: int64 [n]."""
        kf = self.k[layer].view(-1, *self.k.shape[-2:])
        vf = self.v[layer].view(-1, *self.v.shape[-2:])
        kf.index_copy_(0, slots, k.to(kf.dtype))
        vf.index_copy_(0, slots, v.to(vf.dtype))

    def gather(self, layer: int, seq: SequenceKV, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        pages = torch.tensor(seq.pages[: (length + self.page_size - 1) // self.page_size], device=self.k.device)
        k = self.k[layer][pages].reshape(-1, *self.k.shape[-2:])[:length]
        v = self.v[layer][pages].reshape(-1, *self.v.shape[-2:])[:length]
        return k, v
