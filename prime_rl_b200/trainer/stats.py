"""Cross-rank distribution statistics of per-token quantities (entropy, trainer / engine mismatch KL, log
importance ratio ...): mean, median, std, min and max over every loss token of every rank of the step.

The reference gathers the raw per-token tensors of all ranks to every rank and reduces them there
(src/prime_rl/trainer/utils.py:207-283: variable-length all-gather, ``.item()`` per statistic). Here nothing
but sufficient statistics crosses the fabric and nothing is read on the host: every rank folds its tokens into
(count, sum, sum of squares, min, max), the median comes from two rounds of a fixed-width histogram (the
second round refines the bin that holds the middle rank, which pins the median to a 16-millionth of the
value range), each round is one small all-reduce, and the results stay device scalars that join the step's
single device-to-host read.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_BINS = 4096


class TensorStats:
    def __init__(self, group=None):
        self.group = group
        self.values: dict[str, list[torch.Tensor]] = {}

    def add(self, key: str, values: torch.Tensor, mask: torch.Tensor | None = None) -> None:
        """Records the (masked) entries of a 1-D tensor; call with the same keys in the same order on every rank."""
        v = values.detach().float().reshape(-1)
        if mask is not None:
            v = v[mask.reshape(-1)]
        self.values.setdefault(key, []).append(v)

    def _all_reduce(self, t: torch.Tensor, op) -> torch.Tensor:
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def compute(self) -> dict[str, torch.Tensor]:
        """``{key/mean, key/median, key/std, key/min, key/max}`` as 0-dim device tensors; clears the store.
        Keys without any token on any rank give NaN."""
        out: dict[str, torch.Tensor] = {}
        keys = list(self.values)
        if not keys:
            return out
        data = [torch.cat(self.values[k]) if self.values[k] else None for k in keys]
        dev = next((d.device for d in data if d is not None), torch.device("cpu"))
        data = [d if d is not None else torch.empty(0, device=dev) for d in data]
        self.values = {}
        K = len(keys)
        inf = float("inf")
        sums = torch.stack([torch.stack([torch.tensor(float(d.numel()), device=dev), d.sum(), (d * d).sum()])
                            for d in data])                                             # [K, 3]
        lo = torch.stack([d.min() if d.numel() else torch.tensor(inf, device=dev) for d in data])
        hi = torch.stack([d.max() if d.numel() else torch.tensor(-inf, device=dev) for d in data])
        sums = self._all_reduce(sums.double(), dist.ReduceOp.SUM)
        lo = self._all_reduce(lo, dist.ReduceOp.MIN)
        hi = self._all_reduce(hi, dist.ReduceOp.MAX)
        n, s1, s2 = sums[:, 0], sums[:, 1], sums[:, 2]
        mean = s1 / n
        var = ((s2 - n * mean * mean) / (n - 1).clamp_min(1)).clamp_min(0)               # unbiased, as torch.std
        std = torch.where(n > 1, var.sqrt(), torch.full_like(var, float("nan")))
        median = self._median(data, lo, hi, n)
        nan = torch.full_like(mean, float("nan"))
        empty = n == 0
        for i, k in enumerate(keys):
            out[f"{k}/mean"] = torch.where(empty[i], nan[i], mean[i]).float()
            out[f"{k}/median"] = torch.where(empty[i], nan[i].float(), median[i])
            out[f"{k}/std"] = std[i].float()
            out[f"{k}/min"] = torch.where(empty[i], nan[i].float(), lo[i])
            out[f"{k}/max"] = torch.where(empty[i], nan[i].float(), hi[i])
        return out

    def _median(self, data, lo, hi, n) -> torch.Tensor:
        """Lower median (the element of rank floor((n - 1) / 2), what ``torch.median`` returns) of the union of
        all ranks' values, by histogram bisection."""
        K = len(data)
        dev = lo.device
        target = ((n - 1).clamp_min(0) // 2).to(torch.int64)           # 0-based rank of the median element
        lo_k = torch.where(torch.isfinite(lo), lo, torch.zeros_like(lo)).double()
        hi_k = torch.where(torch.isfinite(hi), hi, torch.zeros_like(hi)).double()
        below = torch.zeros(K, dtype=torch.int64, device=dev)          # elements known to lie under the window
        for _ in range(2):
            width = ((hi_k - lo_k) / _BINS).clamp_min(1e-30)
            hist = torch.zeros(K, _BINS, dtype=torch.int64, device=dev)
            for i, d in enumerate(data):
                if d.numel():
                    inside = (d.double() >= lo_k[i]) & (d.double() <= hi_k[i])
                    b = ((d.double() - lo_k[i]) / width[i]).floor().clamp_(0, _BINS - 1).long()[inside]
                    hist[i].scatter_add_(0, b, torch.ones_like(b))
            hist = self._all_reduce(hist, dist.ReduceOp.SUM)
            cum = hist.cumsum(1) + below[:, None]
            idx = (cum > target[:, None]).float().argmax(1)                           # first bin reaching the rank
            prev = torch.where(idx > 0, cum.gather(1, (idx - 1).clamp_min(0)[:, None])[:, 0], below)
            below = prev
            new_lo = lo_k + idx.double() * width
            hi_k = torch.minimum(hi_k, new_lo + width)
            lo_k = new_lo
        # the window is now narrower than float32 resolution for any realistic range: take the smallest actual
        # value inside it (the values of the winning bin are identical on every rank that holds one)
        big = torch.tensor(float("inf"), device=dev)
        cand = torch.stack([torch.where((d.double() >= lo_k[i]) & (d.double() <= hi_k[i]), d, big).min()
                            if d.numel() else big for i, d in enumerate(data)])
        return self._all_reduce(cand, dist.ReduceOp.MIN)
