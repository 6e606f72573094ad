"""Equal-split all-to-all over NVLink peer memory (the sequence <-> head exchange of Ulysses
context parallelism): every rank stores block ``d`` of its input straight into rank ``d``'s
receive buffer with a copy kernel (``csrc/weight_push.cu: weight_copy_kernel``, plain 16-byte
peer stores), then raises an epoch flag there (``csrc/ep_p2p.cu``); the receiver waits for the
flags of all senders (bounded) and reads its own memory. Two receive buffers alternate, and a
sender reuses a buffer only after every peer has reported that it consumed the previous contents.

Takes the place of ``dist.all_to_all_single`` in ``parallel/cp.py`` (the reference's Ulysses
path, src/prime_rl/trainer/models/layers/ulysses_attn.py:53-152, uses NCCL).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _runtime as rt
from .symm import SymmetricBuffer

_K_DATA, _K_CONSUMED = 0, 1


class P2PAllToAll:
    def __init__(self, group, max_bytes_per_block: int, device: torch.device):
        self.group, self.device = group, device
        self.R, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.slot = (int(max_bytes_per_block) + 255) // 256 * 256
        self.buf_bytes = self.R * self.slot
        self.off_flags = 2 * self.buf_bytes
        self.mem = SymmetricBuffer(group, self.off_flags + 256, device, zero=True)
        self.flags = self.mem.local(torch.int32, self.off_flags, 2 * self.R)
        self.p_flags = self.mem.offset_ptrs(self.off_flags)
        self.local = [self.mem.local(torch.uint8, b * self.buf_bytes, self.buf_bytes) for b in range(2)]
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """x: [R, ...] contiguous (block d goes to rank d). Returns [R, ...] (block s came from rank s)."""
        lib, dev, R = rt.lib(), self.device, self.R
        assert x.shape[0] == R and x.is_contiguous()
        nbytes = x[0].numel() * x.element_size()
        if nbytes > self.slot:
            raise ValueError(f"block of {nbytes} bytes exceeds the {self.slot}-byte slots of this exchange")
        self.epoch += 1
        ep, b = self.epoch, self.epoch & 1
        st, stream = rt.status_tensor(dev).data_ptr(), rt.stream_ptr(dev)
        if ep > 2:      # the buffer was last used at epoch ep - 2: wait until every peer has consumed that
            rt.check(lib.prb_ep_wait(self.flags.data_ptr(), R, _K_CONSUMED, ep - 2, st, stream), "prb_ep_wait")
        out = torch.empty_like(x)
        if nbytes % 16 == 0:
            # two launches: push (all destinations, raises the data flags) and receive (waits,
            # copies out of this rank's own buffer, raises the consumed flags)
            p_buf = self.mem.offset_ptrs(0)
            rt.check(lib.prb_a2a_push(x.data_ptr(), p_buf, self.p_flags, nbytes, self.slot, b * self.buf_bytes,
                                      self.done.data_ptr(), self.rank, R, _K_DATA, ep, stream), "prb_a2a_push")
            rt.check(lib.prb_a2a_recv(self.local[b].data_ptr(), out.data_ptr(), self.p_flags, self.flags.data_ptr(),
                                      nbytes, self.slot, self.done.data_ptr(), self.rank, R, _K_DATA, _K_CONSUMED, ep,
                                      st, stream), "prb_a2a_recv")
            return out
        base = b * self.buf_bytes + self.rank * self.slot
        for d in range(R):
            rt.check(lib.prb_weight_push(x[d].data_ptr(), self.mem.ptrs[d] + base, nbytes, stream), "prb_weight_push")
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, R, _K_DATA, ep, stream), "prb_ep_signal")
        rt.check(lib.prb_ep_wait(self.flags.data_ptr(), R, _K_DATA, ep, st, stream), "prb_ep_wait")
        flat = out.view(R, -1).view(torch.uint8) if x.dtype != torch.uint8 else out.view(R, -1)
        flat.copy_(self.local[b].view(R, self.slot)[:, :nbytes])
        rt.check(lib.prb_ep_signal(self.p_flags, self.rank, R, _K_CONSUMED, ep, stream), "prb_ep_signal")
        return out

    def close(self):
        self.mem.close()
