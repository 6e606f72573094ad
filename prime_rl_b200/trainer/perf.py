"""Throughput and MFU accounting.

FLOPs per token = 6 * active matmul parameters + 12 * L * H_q * D * T_attn (the attention
score/value products, with T_attn the mean attended length), the formula of the
reference's perf counter (src/prime_rl/trainer/perf.py:177-213). With LoRA the base weight
gradient is not formed, so the matmul term is 4x instead of 6x of the frozen parameters;
activation recomputation is not counted as useful work.
"""

from __future__ import annotations

import time
from collections import deque

from ..models.config import ModelArch

PEAK_BF16_FLOPS = {"B200": 2.25e15, "H100": 989e12, "H200": 989e12, "A100": 312e12}


def peak_flops(device_name: str) -> float:
    for k, v in PEAK_BF16_FLOPS.items():
        if k in device_name:
            return v
    return 2.25e15


def flops_per_token(arch: ModelArch, seq_len: int, *, lora: bool = False, causal: bool = True) -> float:
    active = arch.param_count(active_only=True, matmul_only=True)
    mm = (4 if lora else 6) * active
    attn = 12 * arch.num_hidden_layers * arch.num_attention_heads * arch.head_dim * seq_len
    if causal:
        attn = attn / 2
    return float(mm + attn)


def count_params(arch: ModelArch) -> tuple[int, int]:
    """(parameters outside the routed experts, parameters of the routed experts): what expert parallelism
    replicates and what it spreads over the ranks."""
    H = arch.hidden_size
    moe_layers = sum(1 for i in range(arch.num_hidden_layers) if arch.is_moe and arch.layer_is_moe(i))
    expert = moe_layers * arch.num_experts * 3 * H * arch.moe_intermediate_size if arch.is_moe else 0
    return arch.param_count() - expert, expert


class PerfCounter:
    def __init__(self, arch: ModelArch, seq_len: int, world_size: int, device_name: str = "B200", lora: bool = False,
                 window: int = 10):
        self.fpt = flops_per_token(arch, seq_len, lora=lora)
        self.world_size, self.peak = world_size, peak_flops(device_name)
        self.samples: deque[tuple[float, int]] = deque(maxlen=window)

    def count_tokens(self, tokens: int) -> None:
        self.samples.append((time.perf_counter(), tokens))

    def throughput(self) -> float | None:
        if len(self.samples) < 2:
            return None
        dt = self.samples[-1][0] - self.samples[0][0]
        toks = sum(t for _, t in list(self.samples)[1:])
        return toks / dt if dt > 0 else None

    def mfu(self, tokens_per_second: float | None = None) -> float | None:
        tps = tokens_per_second if tokens_per_second is not None else self.throughput()
        if tps is None:
            return None
        return 100.0 * tps * self.fpt / (self.world_size * self.peak)
