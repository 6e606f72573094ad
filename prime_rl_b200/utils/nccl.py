"""Topology probe for the library collectives and the peer-memory kernels.

``nvlink_present`` asks NVML (read-only) whether any GPU of the box has an active NVLink;
``configure_nccl_transports`` turns NCCL's P2P and shared-memory transports off when none has
(PCIe-only hosts, VMs with passed-through GPUs: CUDA IPC between such GPUs fails), unless the user
has set the variables; ``peer_memory_usable`` is what the peer-memory paths (EP dispatcher, weight
push, optimizer collectives) check before they map each other's buffers. NVML is injectable so that
the logic is testable without a GPU (reference: src/prime_rl/utils/nccl.py:8-42).
"""

from __future__ import annotations

import os

MAX_LINKS = 18


def nvlink_present(nvml=None) -> bool | None:
    """True / False, or None when NVML cannot be loaded."""
    if nvml is None:
        try:
            import pynvml as nvml
        except ImportError:
            return None
    try:
        nvml.nvmlInit()
    except Exception:
        return None
    try:
        n = nvml.nvmlDeviceGetCount()
        for i in range(n):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            for link in range(MAX_LINKS):
                try:
                    if nvml.nvmlDeviceGetNvLinkState(h, link):
                        return True
                except Exception:
                    break                       # this GPU has no more links
        return False
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass


def configure_nccl_transports(nvml=None, env=None, logger=None) -> bool:
    """Returns True when the transports were switched off."""
    env = os.environ if env is None else env
    if nvlink_present(nvml) is not False:
        return False
    if "NCCL_P2P_DISABLE" in env and "NCCL_SHM_DISABLE" in env:
        return False
    env["NCCL_P2P_DISABLE"] = "1"
    env["NCCL_SHM_DISABLE"] = "1"
    if logger is not None:
        logger.warning("no NVLink between the GPUs: NCCL P2P and SHM transports are off "
                       "(set NCCL_P2P_DISABLE=0 and NCCL_SHM_DISABLE=0 to override)")
    return True


def peer_memory_usable(num_devices: int | None = None) -> bool:
    """Every pair of visible GPUs can map the other's memory."""
    import torch

    if not torch.cuda.is_available():
        return False
    n = torch.cuda.device_count() if num_devices is None else num_devices
    return all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j)
