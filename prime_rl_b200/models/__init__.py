"""Model families, layers and checkpoint-layout conversions."""

from .config import PRESETS, ModelArch, resolve_arch  # noqa: F401
from .layers import SeqInfo  # noqa: F401
from .model import (CausalLM, apply_fp8_training, apply_lora, build_model, freeze_router,  # noqa: F401
                    check_context_parallel, setup_quantization)
