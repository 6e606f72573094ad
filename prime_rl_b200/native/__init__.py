"""ctypes bindings for the in-tree native libraries.

``cuda()`` returns the sm_100a kernel library, ``cpu()`` the C++ CPU optimizer library. Both
raise a clear error when the shared object is missing instead of falling back silently: on
a GPU machine the hand-written kernels are the only implementation of the CUDA path.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from functools import lru_cache
from pathlib import Path

HERE = Path(__file__).resolve().parent
CUDA_LIB = HERE / "libprb200_cuda.so"
CPU_LIB = HERE / "libprb200_cpu.so"

P, I, L, F = c_void_p, c_int, c_longlong, c_float

_CUDA_SIGNATURES = {
    # name: argtypes (restype is always int)
    "prb_bind_device": [I],
    "prb_sm_count": [],
    "prb_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, F, F, P, I, I, I, P, P],
    "prb_gemm_bf16_kgrouped": [P, P, P, I, I, L, L, L, L, I, F, F, P, I, P, P],
    "prb_flash_fwd": [P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, I, I, P, P],
    "prb_symm_alloc": [L, P], "prb_symm_free": [P], "prb_symm_memset": [P, I, L, P],
    "prb_symm_export": [P, P], "prb_symm_import": [P, P], "prb_symm_unmap": [P],
    "prb_ep_hist": [P, P, P, I, I, I, I, I, P],
    "prb_ep_plan": [P, P, I, I, I, I, I, I, I, P, P, P, P, P, P],
    "prb_ep_push": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
    "prb_ep_recv": [P, P, P, P, I, I, I, I, I, I, P, P],
    "prb_ep_push_fp8": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
    "prb_ep_recv_fp8": [P, P, P, P, P, P, I, I, I, I, I, I, P, P],
    "prb_ipc_export_range": [P, P, P], "prb_weight_push": [P, P, L, P],
    "prb_weight_push_fp8": [P, L, P, P, I, I, P],
    "prb_gemm_fp8": [P, P, P, P, P, I, I, I, L, P, I, P, P, P], "prb_act_quant_fp8": [P, L, P, P, I, I, P, P],
    "prb_a2a_push": [P, P, P, L, L, L, P, I, I, I, I, P],
    "prb_a2a_recv": [P, P, P, P, L, L, P, I, I, I, I, I, P, P],
    "prb_ep_wait": [P, I, I, I, P, P],
    "prb_gemm_bf16_reduce_scatter": [P, P, I, I, I, L, L, I, I, F, P, I, I, L, P, P],
    "prb_gemm_bf16_allgather": [P, P, P, P, I, I, I, L, L, I, I, F, I, I, I, P, I, P, P],
    "prb_flash_fwd_gather": [P, P, P, L, P, P, P, I, I, I, I, L, L, F, I, I, I, I, I, P, P, P],
    "prb_sparse_mla_fwd": [P, P, P, P, P, I, I, I, I, F, P, P],
    "prb_gated_norm_fwd": [P, P, P, P, L, I, I, I, F, I, P],
    "prb_gated_norm_bwd": [P, P, P, P, P, P, P, L, I, I, I, F, I, P],
    "prb_conv1d_fwd": [P, P, P, P, P, L, I, I, I, P],
    "prb_sample_gumbel": [P, P, L, L, P, P, I, I, P],
    "prb_sample_truncated": [P, P, P, P, L, L, P, P, P, P, I, I, I, P],
    "prb_conv1d_bwd": [P, P, P, P, P, P, P, P, L, I, I, I, P],
    "prb_rs_pull": [P, L, L, F, P, I, P],
    "prb_ar_add_rmsnorm": [P, P, P, P, P, P, P, I, I, F, I, I, P, P],
    "prb_ag_push": [P, P, L, L, I, I, P],
    "prb_ep_signal": [P, I, I, I, I, P],
    "prb_ep_pull": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
    "prb_gemm_bf16_ext": [P, P, P, I, I, I, L, L, L, I, I, I, F, F, P, I, I, I, P, P, I, L, L, I, P, P],
    "prb_flash_fwd_slice": [P, P, P, P, P, P, I, I, I, I, I, I, I, L, L, L, L, F, I, I, P, P, P],
    "prb_attn_merge": [P, P, P, P, L, I, P],
    "prb_peer_copy": [P, P, L, I, P],
    "prb_slot_pull_reduce": [P, L, L, P, I, P],
    "prb_flash_fwd_block": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, L, L, L, L, F, I, I, P, P, P],
    "prb_flash_bwd_block": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, L, L, L, L, L, L, L, F, I, I, P, P],
    "prb_flash_bwd_slice": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, L, L, L, L, L, L, L, F, I, I, P, P],
    "prb_flash_bwd": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, L, F, I, I, P, P],
    "prb_paged_decode": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P],
    "prb_paged_decode_prefix": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, P, P, I, I, P],
    "prb_lmhead_num_splits": [I, I],
    "prb_lmhead_fwd": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, L, L, I, P, P],
    "prb_lmhead_bwd_dlogits": [P, P, P, P, P, P, P, I, I, I, L, L, L, P, P],
    "prb_rmsnorm_fwd": [P, P, P, P, P, P, L, I, F, P],
    "prb_rmsnorm_bwd_parts": [L],
    "prb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, L, I, P],
    "prb_qknorm_rope": [P, P, P, P, P, P, P, P, L, I, I, L, L, L, F, I, P],
    "prb_glu_fwd": [P, P, P, L, I, L, L, I, F, F, P],
    "prb_glu_bwd": [P, P, P, P, P, L, I, L, L, L, I, F, F, P],
    "prb_sumsq": [P, L, I, P, P],
    "prb_clip_coef": [P, F, P, P, P],
    "prb_adamw": [P, P, P, P, I, P, L, P, F, F, F, F, F, P, P],
    "prb_rl_loss": [P, P, P, P, P, P, L, I, F, F, F, F, P, P],
    "prb_router_topk": [P, P, P, P, P, P, P, L, I, I, I, I, F, P],
    "prb_moe_plan": [P, P, P, P, P, P, P, P, L, I, I, I, I, P],
    "prb_mamba2_step": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "prb_delta_rule_step": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "prb_moe_plan_range": [P, P, P, P, P, P, P, P, L, I, I, I, I, I, P],
    "prb_moe_gather_rows": [P, P, P, P, L, I, I, P, P],
    "prb_qkv_rope_cache": [P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, F, P],
    "prb_moe_route_plan_small": [P, P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, I, F, P],
    "prb_moe_gather_rows_nopad": [P, P, P, P, L, I, I, P, P],
    "prb_glu_fwd_rowmask": [P, P, P, L, I, L, L, I, F, F, P, P],
    "prb_gemm_bf16_rowmask": [P, P, P, I, I, I, L, L, L, I, I, I, F, F, P, I, I, I, P, P, P],
    "prb_gemm_bf16_grouped_arrive": [P, P, P, I, I, I, L, L, L, I, I, P, I, I, P, P, P, P],
    "prb_ep_prepare": [P, P, P, P, P, I, I, I, I, I, P],
    "prb_ep_push_blocks": [P, P, P, P, P, P, P, P, P, L, P, I, I, I, I, I, I, I, P, P],
    "prb_gemm_bf16_splitk": [P, P, P, I, I, I, L, L, L, I, I, F, F, P, L, I, I, P, P],
    "prb_moe_combine": [P, P, P, P, P, L, I, I, P],
    "prb_moe_combine_bwd_w": [P, P, P, P, L, I, I, P],
}


class NativeLibraryMissing(RuntimeError):
    pass


def _load(path: Path, signatures: dict) -> ctypes.CDLL:
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path.name} is not built. Run `python -m prime_rl_b200.native.build` "
            "(needs nvcc / g++); the CUDA path has no eager fallback."
        )
    lib = ctypes.CDLL(str(path))
    for name, argtypes in signatures.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue  # optional symbol; looked up lazily by callers that need it
        fn.argtypes = argtypes
        fn.restype = c_int
    return lib


@lru_cache(maxsize=None)
def cuda() -> ctypes.CDLL:
    return _load(CUDA_LIB, _CUDA_SIGNATURES)


@lru_cache(maxsize=None)
def cpu() -> ctypes.CDLL:
    from .cpu_signatures import CPU_SIGNATURES

    return _load(CPU_LIB, CPU_SIGNATURES)


def cuda_available() -> bool:
    return CUDA_LIB.exists()


def register(name: str, argtypes: list) -> None:
    """Declare the signature of an additional exported symbol (used by optional kernels)."""
    _CUDA_SIGNATURES[name] = argtypes
    if cuda.cache_info().currsize:
        fn = getattr(cuda(), name)
        fn.argtypes = argtypes
        fn.restype = c_int
