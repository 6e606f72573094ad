"""Shared plumbing of the kernel front ends: stream handles, the device status word that
bounded waits report into, and return-code checks."""

from __future__ import annotations

import ctypes

import torch

from .. import native

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free stage (empty barrier)",
    3: "timeout waiting for an accumulator (tmem full)",
    4: "timeout waiting for an accumulator to drain (tmem empty)",
    5: "timeout waiting for a peer flag",
    6: "bad argument",
}

_status: dict[int, torch.Tensor] = {}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    return native.cuda()


def stream_ptr(device: torch.device | None = None) -> int:
    """Current stream handle of ``device``; also binds the device's context to the calling
    thread inside the native library (autograd worker threads start without one)."""
    idx = device.index if device is not None and device.index is not None else torch.cuda.current_device()
    rc = lib().prb_bind_device(idx)
    if rc != 0:
        raise KernelError(f"cannot bind CUDA device {idx} (code {rc})")
    return torch.cuda.current_stream(idx).cuda_stream


_sms: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    idx = device.index if device is not None and device.index is not None else torch.cuda.current_device()
    n = _sms.get(idx)
    if n is None:
        n = _sms[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_tensor(device: torch.device) -> torch.Tensor:
    """One int32 per device; kernels write a non-zero code when a bounded wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device: torch.device | None = None) -> None:
    """Synchronising read of the status word; raises when a kernel reported a failure."""
    devs = [device.index] if device is not None and device.index is not None else list(_status)
    for idx in devs:
        t = _status.get(idx)
        if t is None:
            continue
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise KernelError(f"device {idx}: {STATUS_NAMES.get(code, code)}")


_launches = 0


def launch_count() -> int:
    """Number of native kernel-launching calls issued so far by this process."""
    return _launches


def check(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")
