"""The two collectives of the sharded optimizer over NVLink peer memory: the flat fp32 gradient
buffer and the flat compute-dtype parameter buffer of a group live in one symmetric allocation,
so that

``reduce_scatter``  every rank sums its own slice of all ranks' gradient buffers with peer loads,
                    scales it and writes its fp32 shard (``csrc/ep_p2p.cu: rs_pull_kernel``);
``all_gather``      after the update every rank stores its new parameter slice into the same place
                    of every peer's parameter buffer (``ag_push_kernel``).

Epoch flags in peer memory order the steps (gradients complete before anybody pulls, everybody
has pulled before gradients are zeroed, all slices landed before the next forward). Takes the
place of FSDP2's bucket reduce-scatter with cast / scale and parameter all-gather
(src/prime_rl/trainer/model.py:470-559) for the ZeRO-style sharding of ``trainer/optim.py``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _runtime as rt
from .symm import SymmetricBuffer

_K_GRADS, _K_PULLED, _K_PUSHED = 0, 1, 2


class P2PShardCollectives:
    def __init__(self, group, flat_numel: int, flat_dtype: torch.dtype, device: torch.device):
        self.group, self.device = group, device
        self.R, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.R > 8:
            raise ValueError("at most 8 ranks (one NVSwitch box)")
        item = torch.empty(0, dtype=flat_dtype).element_size()
        self.off_grad = (flat_numel * item + 255) // 256 * 256
        self.off_flags = self.off_grad + (flat_numel * 4 + 255) // 256 * 256
        self.mem = SymmetricBuffer(group, self.off_flags + 256, device, zero=True)
        self.flat = self.mem.local(flat_dtype, 0, flat_numel)
        self.grad = self.mem.local(torch.float32, self.off_grad, flat_numel)
        self.flags = self.mem.local(torch.int32, self.off_flags, 3 * self.R)
        self.p_flat = self.mem.offset_ptrs(0)
        self.p_grad = self.mem.offset_ptrs(self.off_grad)
        self.p_flags = self.mem.offset_ptrs(self.off_flags)
        self.item, self.epoch = item, 0

    def _barrier(self, kind: int) -> None:
        lib, st, stream = rt.lib(), rt.status_tensor(self.device).data_ptr(), rt.stream_ptr(self.device)
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, self.R, kind, self.epoch, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), self.R, kind, self.epoch, st, stream), "prb_ep_wait")

    def reduce_scatter(self, out: torch.Tensor, lo: int, scale: float = 1.0) -> None:
        """``out [n]`` fp32 = scale * sum over ranks of ``grad[lo:lo + n]``."""
        self.epoch += 1
        self._barrier(_K_GRADS)
        rt.check(rt.lib().prb_rs_pull(self.p_grad, lo, out.numel(), float(scale), out.data_ptr(), self.R,
                                      rt.stream_ptr(self.device)), "prb_rs_pull")
        self._barrier(_K_PULLED)

    def all_gather(self, lo: int, n: int) -> None:
        """Publishes ``flat[lo:lo + n]`` (already updated in place) to every peer's ``flat``."""
        src = self.flat[lo:lo + n]
        rt.check(rt.lib().prb_ag_push(src.data_ptr(), self.p_flat, lo * self.item, n * self.item, self.rank, self.R,
                                      rt.stream_ptr(self.device)), "prb_ag_push")
        self._barrier(_K_PUSHED)

    def close(self) -> None:
        self.mem.close()
