"""Orchestrator -> trainer wire format: msgpack, positional (array-like) structs. Fields are
append-only so that the positional layout of earlier fields never moves. Field order and
meaning follow the reference's ``transports/batch/types.py:7-130``, which makes batch files
and ZMQ frames interchangeable between the two implementations.
"""

from __future__ import annotations

import msgspec
import numpy as np
import torch


class EncodedTensor(msgspec.Struct, array_like=True, gc=False):
    dtype: str
    shape: list[int]
    data: bytes


class RoutedExperts(msgspec.Struct, array_like=True, gc=False, omit_defaults=True):
    data: bytes
    shape: list[int]  # [seq_len, layers, topk]
    dtype: str


class SamplingMask(msgspec.Struct, array_like=True, gc=False, omit_defaults=True):
    ids: bytes      # flat int32 token ids
    counts: bytes   # int32 count per token position; len(ids) == 4 * sum(counts)


class TrainingSample(msgspec.Struct, array_like=True, gc=False, omit_defaults=True):
    """One rollout branch; all per-token arrays share ``len(token_ids)``."""

    token_ids: list[int]
    mask: list[bool]
    logprobs: list[float]
    temperatures: list[float]
    env_name: str
    ref_logprobs: list[float] | None = None
    mm_kwargs: dict[str, EncodedTensor] | None = None
    routed_experts: RoutedExperts | None = None
    mm_token_type_ids: list[int] | None = None
    rl_weights: list[float] | None = None
    ce_weights: list[float] | None = None
    ref_kl_weights: list[float] | None = None
    advantages: list[float] | None = None
    sampling_mask: SamplingMask | None = None
    trace_id: str | None = None
    branch_index: int | None = None


class MicroBatch(msgspec.Struct, array_like=True, gc=False, omit_defaults=True):
    """One packed row for one trainer data-parallel rank."""

    input_ids: list[int]
    loss_mask: list[bool]
    advantages: list[float]
    inference_logprobs: list[float]
    position_ids: list[int]
    sequence_lengths: list[int]
    temperatures: list[float]
    env_names: list[str]
    seq_lens: list[int]
    ref_logprobs: list[float] | None = None
    routed_experts: RoutedExperts | None = None
    mm_kwargs: dict[str, EncodedTensor] | None = None
    mm_token_type_ids: list[int] | None = None
    rl_weights: list[float] | None = None
    ce_weights: list[float] | None = None
    ref_kl_weights: list[float] | None = None
    sampling_mask: SamplingMask | None = None
    trace_ids: list[str] | None = None
    branch_indices: list[int] | None = None


_encoder = msgspec.msgpack.Encoder()
_decoder = msgspec.msgpack.Decoder(list[MicroBatch])


def encode_micro_batches(mbs: list[MicroBatch]) -> bytes:
    return _encoder.encode(mbs)


def decode_micro_batches(buf: bytes) -> list[MicroBatch]:
    return _decoder.decode(buf)


def encode_tensor(t: torch.Tensor) -> EncodedTensor:
    """Any CPU tensor -> wire form (bf16 travels as its raw 16-bit words)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return EncodedTensor(dtype="bfloat16", shape=list(t.shape), data=t.view(torch.int16).numpy().tobytes())
    arr = t.numpy()
    return EncodedTensor(dtype=str(arr.dtype), shape=list(arr.shape), data=arr.tobytes())


def decode_tensor(e: EncodedTensor) -> torch.Tensor:
    if e.dtype == "bfloat16":
        arr = np.frombuffer(e.data, dtype=np.int16).reshape(e.shape)
        return torch.from_numpy(arr.copy()).view(torch.bfloat16)
    arr = np.frombuffer(e.data, dtype=np.dtype(e.dtype)).reshape(e.shape)
    return torch.from_numpy(arr.copy())


def encode_routed_experts(arr: np.ndarray) -> RoutedExperts:
    return RoutedExperts(data=arr.tobytes(), shape=list(arr.shape), dtype=str(arr.dtype))


def decode_routed_experts(re: RoutedExperts) -> torch.Tensor:
    arr = np.frombuffer(re.data, dtype=np.dtype(re.dtype)).reshape(re.shape)
    return torch.from_numpy(arr.astype(np.int32))


def decode_sampling_mask(sm: SamplingMask, num_tokens: int) -> torch.Tensor:
    """-> int32 [T, Kmax] padded with -1."""
    counts = np.frombuffer(sm.counts, dtype=np.int32)
    ids = np.frombuffer(sm.ids, dtype=np.int32)
    kmax = int(counts.max()) if counts.size else 0
    out = np.full((num_tokens, max(kmax, 1)), -1, dtype=np.int32)
    off = 0
    for t, c in enumerate(counts[:num_tokens]):
        if c:
            out[t, :c] = ids[off:off + c]
            off += c
    return torch.from_numpy(out)
