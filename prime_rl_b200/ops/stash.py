"""Selective activation recomputation: a checkpointed decoder layer is re-run in the backward pass, but the
outputs of its expensive operators (GEMMs, grouped GEMMs; attention has its own cache in ``ops/attention.py``)
are kept from the first pass, so the re-run only repeats the cheap element-wise work around them.

The operators here are ctypes launches inside ``autograd.Function``s, invisible to PyTorch's dispatcher-based
selective-checkpoint policies, so the bookkeeping is explicit: while a layer runs under ``stash.layer(idx)``
every participating operator either *records* its output (first pass) or *replays* the recorded tensor in
call order without launching its kernel (second pass of the same layer index). The autograd node is built in
both passes; only the forward arithmetic is skipped.

Role of the reference's ``selective`` mode (src/prime_rl/trainer/activation_checkpointing.py:31-106: whole-block
checkpointing that saves matmul / attention / collective outputs by operator name).
"""

from __future__ import annotations

import contextlib

import torch

# operator classes that can be kept, and the reference's operator / namespace names that select them
KINDS = ("mm", "grouped_mm", "attention")
_ALIASES = {
    "mm": {"mm", "aten::mm", "aten::linear", "aten::addmm", "aten::bmm", "aten::_scaled_mm", "aten::_scaled_mm_v2",
           "prime_rl::fp8_blockwise_mm"},
    "grouped_mm": {"grouped_mm", "aten::_grouped_mm", "aten::_scaled_grouped_mm", "prime_rl::grouped_fp8_gemm"},
    "attention": {"attention", "flash_attn", "flash_attn_3", "prime_rl_ring", "prime_rl::sparse_mla",
                  "prime_rl::dsv4_sparse_attn", "aten::_flash_attention_forward",
                  "aten::_scaled_dot_product_flash_attention", "aten::_scaled_dot_product_efficient_attention",
                  "aten::_scaled_dot_product_cudnn_attention", "aten::_efficient_attention_forward",
                  "aten::_scaled_dot_product_attention_math"},
}


def kinds_from_targets(targets: list[str] | None) -> set[str]:
    """``None``: everything that can be kept. Otherwise the classes named by this framework's own words
    (``mm``, ``grouped_mm``, ``attention``) or by the operator names the reference's configs use."""
    if targets is None:
        return set(KINDS)
    out = {kind for kind, names in _ALIASES.items() if names & set(targets)}
    return out


class OpStash:
    def __init__(self, kinds: set[str]):
        self.kinds = set(kinds)
        self.store: dict[int, list[torch.Tensor]] = {}
        self._mode: str | None = None
        self._queue: list[torch.Tensor] = []
        self.stats = {"recorded": 0, "replayed": 0}

    @contextlib.contextmanager
    def layer(self, idx: int):
        """First entry for ``idx`` records, the next one replays and forgets."""
        global _ACTIVE
        prev = _ACTIVE
        if idx in self.store:
            self._mode, self._queue = "replay", self.store.pop(idx)
        else:
            self._mode, self._queue = "record", []
        _ACTIVE = self
        try:
            yield
        finally:
            _ACTIVE = prev
            if self._mode == "record":
                self.store[idx] = self._queue
            elif self._queue:
                raise RuntimeError(f"{len(self._queue)} stashed outputs of layer {idx} were not consumed by its "
                                   "recomputation: the two passes took different paths")
            self._mode, self._queue = None, []

    def run(self, kind: str, compute):
        """``compute()`` on the first pass (result kept), the kept tensor on the second."""
        if kind not in self.kinds or self._mode is None:
            return compute()
        if self._mode == "record":
            y = compute()
            # an alias without autograd history: the operator's own output object gets the first pass's graph
            # attached, and keeping that alive would keep every activation the checkpoint is meant to drop
            self._queue.append(y.detach())
            self.stats["recorded"] += 1
            return y
        self.stats["replayed"] += 1
        return self._queue.pop(0)


_ACTIVE: OpStash | None = None


def active() -> bool:
    return _ACTIVE is not None and _ACTIVE._mode is not None


def run(kind: str, compute):
    """Entry point for operators: keeps / replays ``compute()``'s result when a stash is active."""
    st = _ACTIVE
    if st is None:
        return compute()
    return st.run(kind, compute)
