"""Kernel front ends. Each op runs the hand-written sm_100a kernel for CUDA bf16 tensors
and a plain PyTorch implementation otherwise (CPU tests, oracles)."""

from .activation import RELU2, SWIGLU, SWIGLU_CLAMPED, glu, glu_ref  # noqa: F401
from .matmul import gemm, gemm_ref, grouped_gemm_ref, grouped_linear, linear  # noqa: F401
from .lm_head import (fused_logprob_entropy, logprob_entropy_ref, replay_sampling_mask,  # noqa: F401
                      softcapped_logprob_entropy)
from .norm import add_rms_norm, rms_norm, rms_norm_ref  # noqa: F401
from .rope import inv_freq, qknorm_rope, qknorm_rope_ref, qkv_norm_rope, qkv_rope_to_cache  # noqa: F401
