"""Activation offloading: tensors saved for backward are moved to pinned host memory on a side
stream during the forward pass and brought back shortly before their backward needs them
(``model.ac_offloading``; reference: src/prime_rl/utils/act_offloading.py, a torchtune-style
``saved_tensors_hooks`` context).

Small tensors (< ``min_bytes``), parameters and non-CUDA tensors stay where they are. At most
``max_inflight`` device copies are kept alive waiting for their transfer to finish.
"""

from __future__ import annotations

import torch


class OffloadActivations(torch.autograd.graph.saved_tensors_hooks):
    def __init__(self, pin_memory: bool = True, max_inflight: int = 5, min_bytes: int = 1 << 20):
        self.pin, self.max_inflight, self.min_bytes = pin_memory, max_inflight, min_bytes
        self.stream: torch.cuda.Stream | None = None
        self.inflight: list[tuple[torch.cuda.Event, torch.Tensor]] = []
        self.bytes_offloaded = 0

        def pack(t: torch.Tensor):
            if (not t.is_cuda) or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < self.min_bytes:
                return t
            if self.stream is None:
                self.stream = torch.cuda.Stream(device=t.device)
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.pin)
            self.stream.wait_stream(torch.cuda.current_stream(t.device))
            with torch.cuda.stream(self.stream):
                host.copy_(t, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            # keep the device tensor alive until its copy is done, but not longer
            self.inflight.append((ev, t))
            while len(self.inflight) > self.max_inflight:
                e, _ = self.inflight.pop(0)
                e.synchronize()
            self.bytes_offloaded += t.numel() * t.element_size()
            return ("offloaded", host, t.device, ev)

        def unpack(obj):
            if not (isinstance(obj, tuple) and len(obj) == 4 and obj[0] == "offloaded"):
                return obj
            _, host, dev, ev = obj
            ev.synchronize()
            return host.to(dev, non_blocking=True)

        super().__init__(pack, unpack)

    def __exit__(self, *a):
        for e, _ in self.inflight:
            e.synchronize()
        self.inflight.clear()
        return super().__exit__(*a)
