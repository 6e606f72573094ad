"""Symmetric device memory: every rank of a process group allocates the same number of bytes
and maps all peers' allocations into its own address space (CUDA IPC, one process per GPU on one
NVSwitch box). Kernels take the table of peer pointers and use plain loads / stores on them.

The reference gets the same capability from ``torch.distributed._symmetric_memory`` inside
DeepEP / NCCL (src/prime_rl/trainer/distributed/deepep.py); here it is a 60-line layer over
``cudaIpcGetMemHandle`` / ``cudaIpcOpenMemHandle`` so that the hand-written kernels own the
data path.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _runtime as rt


class _DevMem:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``; ``ptrs[i]`` is rank i's buffer as
    seen from this process (own allocation at index ``rank``)."""

    def __init__(self, group, nbytes: int, device: torch.device, zero: bool = True):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self.device = device
        lib = rt.lib()
        rt.stream_ptr(device)            # binds the device to this thread for the library's runtime
        own = ctypes.c_void_p()
        if lib.prb_symm_alloc(self.nbytes, ctypes.byref(own)) != 0:
            raise RuntimeError(f"symmetric allocation of {self.nbytes} bytes failed")
        self._own = own.value
        if zero:
            lib.prb_symm_memset(self._own, 0, self.nbytes, rt.stream_ptr(device))
            torch.cuda.synchronize(device)
        handle = (ctypes.c_ubyte * 64)()
        if lib.prb_symm_export(self._own, handle) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs: list[int] = []
        self._mapped: list[int] = []
        # Ranks map their peers one after the other: the first mapping of a peer GPU also switches on peer access
        # inside the driver, and eight processes doing that at the same moment is the one thing at start-up that
        # grows with the rank count.
        failed = None
        for turn in range(self.world):
            if turn == self.rank:
                for i, h in enumerate(handles):
                    if i == self.rank:
                        self.ptrs.append(self._own)
                        continue
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    peer = ctypes.c_void_p()
                    if lib.prb_symm_import(buf, ctypes.byref(peer)) != 0:
                        failed = i
                        break
                    self.ptrs.append(peer.value)
                    self._mapped.append(peer.value)
            dist.barrier(group=group)
        if failed is not None:
            raise RuntimeError(f"cudaIpcOpenMemHandle for rank {failed} failed (no peer access between the GPUs?)")
        self.c_ptrs = (ctypes.c_void_p * self.world)(*self.ptrs)     # host table handed to the launchers
        self._local = torch.as_tensor(_DevMem(self._own, self.nbytes), device=device)
        dist.barrier(group=group)        # nobody touches a peer before everybody has mapped it

    def local(self, dtype: torch.dtype, offset: int = 0, numel: int | None = None) -> torch.Tensor:
        """Tensor over a range of this rank's own buffer. Every call makes a tensor with its own
        storage object, so in-place writes to one range do not touch autograd's version counter
        of tensors over another range."""
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = self.nbytes - offset if numel is None else numel * item
        assert offset % 16 == 0 and offset + nbytes <= self.nbytes
        self._keep = getattr(self, "_keep", [])
        mem = _DevMem(self._own + offset, nbytes)
        self._keep.append(mem)
        return torch.as_tensor(mem, device=self.device).view(dtype)

    def offset_ptrs(self, offset: int):
        """Host table of ``ptr + offset`` for every rank."""
        return (ctypes.c_void_p * self.world)(*[p + offset for p in self.ptrs])

    def close(self):
        lib = rt.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._mapped:
            lib.prb_symm_unmap(p)
        self._mapped = []
        if self._own:
            self._local = None
            lib.prb_symm_free(self._own)
            self._own = 0
