"""Peer-memory weight transport: the trainer writes new parameter values straight into the
engine's parameter storage over NVLink (``csrc/weight_push.cu``), optionally quantising to
block-scaled fp8 on the way.

Engine side (``P2PWeightPort``): once, export every parameter's storage with CUDA IPC and write
``<run_dir>/broadcasts/p2p_manifest_<replica>.json`` (name -> handle, byte offset, shape,
dtype; for ``quantize = "fp8"`` also the handles of the e4m3 payload and fp32 scale buffers the
port allocates). Parameters never move afterwards, so the manifest stays valid for the run.

Trainer side (``P2PWeightSender``): after the usual marker-file handshake (the engine is paused
once ``.receiver_ready`` exists) map the handles (cached), launch one push kernel per tensor,
synchronise, and let the base class touch ``.finished``. With several engine replicas trainer
rank r serves replicas r, r + world, ...; replicated parameters need no gather, and an
expert-parallel trainer has every rank write its own expert range at its offset of the engine's stack.

Same role as the reference's NCCL / NIXL transports (src/prime_rl/transports/weights/nccl.py,
nixl.py) for engines on the same NVSwitch box as the trainer.
"""

from __future__ import annotations

import ctypes
import json
import time
from pathlib import Path

import torch

from ...ops import _runtime as rt
from ...utils.logger import get_logger
from ...utils.pathing import get_broadcast_dir
from . import FINISHED, WeightSender

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def manifest_path(run_dir: Path, replica: int) -> Path:
    return get_broadcast_dir(run_dir) / f"p2p_manifest_{replica}.json"


def _export(t: torch.Tensor) -> dict:
    handle = (ctypes.c_ubyte * 64)()
    off = ctypes.c_longlong()
    rc = rt.lib().prb_ipc_export_range(t.data_ptr(), handle, ctypes.byref(off))
    if rc != 0:
        raise RuntimeError(f"cannot export device memory over IPC (code {rc})")
    return {"handle": bytes(handle).hex(), "offset": off.value}


class P2PWeightPort:
    """Engine side. ``quantize``: ``None`` (values land in the live bf16 parameters) or ``"fp8"``
    (2-D weights land as e4m3 + 128 x 128 scales in buffers owned by the port, other tensors as
    they are; ``dequantize_into_model`` refreshes the live parameters from them)."""

    def __init__(self, model, run_dir: Path | None, replica: int = 0, quantize: str | None = None,
                 tp: tuple | None = None):
        """``run_dir=None``: build the manifest only (``self.manifest``), write no file — for callers that
        hand it to the sender through another channel. ``tp = (rank, size[, experts_by_index])``: this process
        holds one tensor-parallel shard of the engine; the manifest says so and the sender slices what it pushes."""
        self.model, self.replica, self.quantize = model, replica, quantize
        self.tp = tp
        self.run_dir = Path(run_dir) if run_dir is not None else None
        self.params = dict(model.named_parameters())
        dev = next(model.parameters()).device
        rt.stream_ptr(dev)
        # An engine that serves from fp8 copies owns (payload, scales) buffers per projection: the push lands
        # in those, nothing is copied or re-quantised on this side afterwards.
        self.live_fp8: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}
        if quantize == "fp8":
            for mname, mod in model.named_modules():
                f8 = getattr(mod, "fp8", None)
                if isinstance(f8, tuple):
                    self.live_fp8[f"{mname}.weight"] = f8
                elif isinstance(f8, dict):
                    for leaf, pair in f8.items():
                        self.live_fp8[f"{mname}.{leaf}"] = pair
        self.fp8: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}
        entries = {}
        for name, p in self.params.items():
            live = self.live_fp8.get(name)
            if live is not None:
                q, s_ = live
                K = q.shape[-1]
                N = q.numel() // K
                shape = list(p.shape) if p.numel() else list(q.shape)
                entries[name] = {"shape": shape, "dtype": "bfloat16",
                                 "fp8": {"q": _export(q), "scales": _export(s_), "rows": N, "cols": K}}
                continue
            if p.numel() == 0:
                continue
            assert p.is_contiguous(), name
            e = {"shape": list(p.shape), "dtype": str(p.dtype).replace("torch.", ""), **_export(p.data)}
            if quantize == "fp8" and p.dim() >= 2 and p.shape[-1] % 2 == 0 and p.dtype == torch.bfloat16:
                K = p.shape[-1]
                N = p.numel() // K
                q = torch.empty(N, K, dtype=torch.uint8, device=dev)
                s_ = torch.empty((N + 127) // 128, (K + 127) // 128, dtype=torch.float32, device=dev)
                self.fp8[name] = (q, s_)
                e["fp8"] = {"q": _export(q), "scales": _export(s_), "rows": N, "cols": K}
            entries[name] = e
        self.manifest = {"device": dev.index or 0, "quantize": quantize, "params": entries,
                         "tp": list(tp) if tp is not None else None}
        if self.run_dir is not None:
            path = manifest_path(self.run_dir, replica)
            path.parent.mkdir(parents=True, exist_ok=True)
            tmp = path.with_suffix(".tmp")
            tmp.write_text(json.dumps(self.manifest))
            tmp.replace(path)

    def wait_finished(self, step_dir: Path, timeout: float = 1200.0) -> None:
        t0 = time.monotonic()
        while not (Path(step_dir) / FINISHED).exists():
            if time.monotonic() - t0 > timeout:
                raise TimeoutError(f"weight push into {step_dir} did not finish after {timeout}s")
            time.sleep(0.01)
        torch.cuda.synchronize()

    def dequantize_into_model(self) -> None:
        """fp8 mode: live bf16 parameter = e4m3 payload x block scale (projections that serve straight
        from the pushed fp8 buffers need nothing; a bf16 copy they still keep is refreshed too)."""
        both = dict(self.fp8)
        both.update({n: pair for n, pair in self.live_fp8.items() if self.params[n].numel() > 0})
        for name, (q, s) in both.items():
            p = self.params[name]
            q = q.reshape(-1, q.shape[-1])
            s = s.reshape(-1, s.shape[-1])
            N, K = q.shape
            w = q.view(torch.float8_e4m3fn).float()
            sc = s.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
            p.data.copy_((w * sc).view(p.shape))

    def receive_into(self, engine, step_dir: Path | None = None) -> None:
        """Called while the engine is paused; returns when the trainer's kernels are done."""
        if step_dir is None:
            steps = sorted((d for d in get_broadcast_dir(self.run_dir).glob("step_*")),
                           key=lambda d: int(d.name[5:]))
            step_dir = steps[-1]
        self.wait_finished(step_dir)
        if self.quantize == "fp8":
            self.dequantize_into_model()
        engine.cache.blocks.clear_prefix_cache()
        engine.policy_version += 1


class _Mapped:
    """IPC mappings of one process, keyed by handle bytes (a block is mapped once)."""

    def __init__(self):
        self.base: dict[str, int] = {}

    def ptr(self, entry: dict) -> int:
        h = entry["handle"]
        if h not in self.base:
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(bytes.fromhex(h))
            out = ctypes.c_void_p()
            if rt.lib().prb_symm_import(buf, ctypes.byref(out)) != 0:
                raise RuntimeError("cudaIpcOpenMemHandle failed (engine and trainer GPUs need peer access)")
            self.base[h] = out.value
        return self.base[h] + entry["offset"]

    def close(self):
        for p in self.base.values():
            rt.lib().prb_symm_unmap(p)
        self.base = {}


def push_state(named_tensors: dict[str, torch.Tensor], manifest: dict, mapped: _Mapped,
               first_expert: dict[str, int] | None = None) -> int:
    """Launches the push kernels on the current stream; returns the bytes written to the peer.

    ``first_expert``: for an expert-parallel trainer, name -> index of the first expert of this
    rank's ``[E / ep, ...]`` slice; the slice lands at that offset of the engine's full stack."""
    lib = rt.lib()
    total = 0
    for name, e in manifest["params"].items():
        t = named_tensors.get(name)
        if t is None:
            continue
        t = t.detach()
        lo = (first_expert or {}).get(name)
        if lo is None:
            if list(t.shape) != e["shape"]:
                raise ValueError(f"{name}: trainer shape {list(t.shape)} != engine shape {e['shape']}")
        else:
            if list(t.shape[1:]) != e["shape"][1:] or lo + t.shape[0] > e["shape"][0]:
                raise ValueError(f"{name}: expert slice {list(t.shape)} at {lo} does not fit engine shape {e['shape']}")
        dev = t.device
        stream = rt.stream_ptr(dev)
        if "fp8" in e and manifest.get("quantize") == "fp8" and t.dtype == torch.bfloat16:
            f = e["fp8"]
            rows, row0 = f["rows"], 0
            if lo is not None:
                per = f["rows"] // e["shape"][0]              # rows of the 2-D view per expert
                rows, row0 = t.shape[0] * per, lo * per
                if row0 % 128 or (rows % 128 and row0 + rows != f["rows"]):
                    raise ValueError(f"{name}: expert slice is not aligned to the 128-row scale blocks")
            t2 = t.reshape(rows, f["cols"])
            t2 = t2 if t2.is_contiguous() else t2.contiguous()
            scale_cols = (f["cols"] + 127) // 128
            rt.check(lib.prb_weight_push_fp8(t2.data_ptr(), t2.stride(0), mapped.ptr(f["q"]) + row0 * f["cols"],
                                             mapped.ptr(f["scales"]) + 4 * (row0 // 128) * scale_cols,
                                             rows, f["cols"], stream), "prb_weight_push_fp8")
            total += rows * f["cols"] + 4 * ((rows + 127) // 128) * scale_cols
        else:
            src = t.to(_DTYPES[e["dtype"]]) if str(t.dtype).replace("torch.", "") != e["dtype"] else t
            src = src if src.is_contiguous() else src.contiguous()
            nbytes = src.numel() * src.element_size()
            off = 0 if lo is None else lo * (nbytes // t.shape[0])
            rt.check(lib.prb_weight_push(src.data_ptr(), mapped.ptr(e) + off, nbytes, stream), "prb_weight_push")
            total += nbytes
    return total


class P2PWeightSender(WeightSender):
    def __init__(self, config, run_dir: Path, world):
        super().__init__(config, run_dir, world, require_ack=True)
        self.run_dir = Path(run_dir)
        self.mapped = _Mapped()
        self.manifests: dict[int, dict] = {}
        self.num_replicas = int(getattr(config, "inference_world_size", 1) or 1)

    def _manifest(self, replica: int) -> dict:
        if replica not in self.manifests:
            path = manifest_path(self.run_dir, replica)
            t0 = time.monotonic()
            while not path.exists():
                if time.monotonic() - t0 > self.config.timeout:
                    raise TimeoutError(f"engine replica {replica} never published {path}")
                time.sleep(0.05)
            self.manifests[replica] = json.loads(path.read_text())
        return self.manifests[replica]

    def _broadcast(self, model, step: int, d: Path) -> None:
        from ...models.convert import expert_parallel_info, is_expert_sharded_key

        tensors = dict(model.named_parameters())
        pushed = 0
        t0 = time.monotonic()
        info = expert_parallel_info(model)
        if info is not None:
            # every rank of the exporting ep group writes the experts it owns into every replica; the
            # replicated tensors of replica i come from the group's rank i % ep
            if info["writer"]:
                lo = info["ep_rank"] * info["local_experts"]
                sliced = {n: t for n, t in tensors.items() if is_expert_sharded_key(n)}
                dense = {n: t for n, t in tensors.items() if n not in sliced}
                for replica in range(self.num_replicas):
                    man = self._manifest(replica)
                    pushed += push_state(sliced, man, self.mapped, first_expert={n: lo for n in sliced})
                    if replica % info["ep"] == info["ep_rank"]:
                        pushed += push_state(dense, man, self.mapped)
        else:
            for replica in range(self.world.rank, self.num_replicas, max(1, self.world.world_size)):
                man = self._manifest(replica)
                src = tensors
                if man.get("tp"):
                    # the target process holds one tensor-parallel shard: send it its slices
                    from ...engine.tp import shard_tensor

                    r, size, *rest = man["tp"]
                    by_expert = bool(rest and rest[0])      # the engine splits its experts by index, not by width
                    src = {n: shard_tensor(n, t.detach(), model.arch, r, size, by_expert) for n, t in tensors.items()}
                pushed += push_state(src, man, self.mapped)
        torch.cuda.synchronize()
        if pushed:
            dt = time.monotonic() - t0
            get_logger().info(f"weight push step {step}: {pushed / 2**30:.2f} GiB in {dt * 1e3:.1f} ms "
                              f"({pushed / dt / 1e9:.0f} GB/s)")
