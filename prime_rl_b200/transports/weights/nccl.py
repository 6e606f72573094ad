"""Library-baseline in-memory weight transport: trainer rank 0 broadcasts the model layer by
layer to every engine process over a dedicated process group (NCCL on GPUs, gloo on CPU) —
the data path of the reference's NCCL transport (src/prime_rl/transports/weights/nccl.py:30-233,
inference/vllm/worker/nccl.py:28-132): per layer one metadata message (names, shapes, dtypes)
and one flat tensor per dtype.

The group is separate from the trainer's own default group: rank 0 is the trainer master,
ranks 1..N the engine workers; rendezvous through a TCP store at ``host:port``.
"""

from __future__ import annotations

import datetime
import pickle
import re
from pathlib import Path

import torch
import torch.distributed as dist

from ...models import convert
from ...utils.logger import get_logger
from . import WeightSender


def _new_group(host: str, port: int, rank: int, world_size: int, timeout: int, device: torch.device):
    store = dist.TCPStore(host, port, world_size, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=timeout), wait_for_workers=False)
    backend = "nccl" if device.type == "cuda" else "gloo"
    from torch.distributed.distributed_c10d import ProcessGroup

    prefix = dist.PrefixStore("weights", store)
    if backend == "gloo":
        pg = dist.ProcessGroupGloo(prefix, rank, world_size, datetime.timedelta(seconds=timeout))
    else:
        from ...utils.nccl import configure_nccl_transports

        configure_nccl_transports()          # PCIe-only hosts: NCCL must not try CUDA IPC between the GPUs
        opts = dist.ProcessGroupNCCL.Options()
        pg = dist.ProcessGroupNCCL(prefix, rank, world_size, opts)
    return pg, store


def _broadcast(pg, tensor: torch.Tensor, src: int = 0) -> None:
    opts = dist.BroadcastOptions()
    opts.rootRank = src
    opts.rootTensor = 0
    pg.broadcast([tensor], opts).wait()


def layer_groups(names: list[str]) -> list[list[str]]:
    """One group per decoder layer plus one for everything else, in a stable order."""
    groups: dict[str, list[str]] = {}
    for n in names:
        m = re.match(r"((?:model|backbone|language_model|model\.language_model)\.layers\.\d+)\.", n)
        groups.setdefault(m.group(1) if m else "_other", []).append(n)
    return list(groups.values())


class NCCLWeightSender(WeightSender):
    def __init__(self, config, run_dir: Path, world):
        super().__init__(config, run_dir, world, require_ack=True)
        self.pg = None
        self._connecting = None
        self._connect_error: BaseException | None = None

    def connect_in_background(self, device) -> None:
        """Starts the rendezvous with the engines right away (from the trainer's set-up). The engines join when the
        orchestrator posts ``/init_broadcaster``, which it does before it produces the first batch: a trainer that
        only connected at its first broadcast (after its first step) would wait for a batch that the orchestrator
        cannot produce while its request to the engines is still waiting for the trainer."""
        if not self.world.is_master or self.pg is not None or self._connecting is not None:
            return
        import threading

        def run():
            try:
                if device.type == "cuda":
                    torch.cuda.set_device(device)
                self.pg, self.store = _new_group(self.config.host, self.config.port, 0,
                                                 self.config.inference_world_size + 1, self.config.timeout, device)
            except BaseException as e:
                # The engines are (or will be) waiting in the same rendezvous and the orchestrator behind them, so no
                # batch would ever reach this trainer: end the main thread now instead of at a first broadcast that
                # never comes. The launcher sees the exit and takes the run down.
                self._connect_error = e
                get_logger().error(f"the weight-broadcast group could not be formed: {type(e).__name__}: {e}")
                import _thread

                _thread.interrupt_main()

        self._connecting = threading.Thread(target=run, name="weight-broadcast-connect", daemon=True)
        self._connecting.start()

    def _connect(self, device):
        if not self.world.is_master:
            return
        if self._connecting is not None:
            self._connecting.join()
            self._connecting = None
            if self._connect_error is not None:
                raise RuntimeError("the weight-broadcast group could not be formed") from self._connect_error
        if self.pg is None:
            self.pg, self.store = _new_group(self.config.host, self.config.port, 0,
                                             self.config.inference_world_size + 1, self.config.timeout, device)

    def _broadcast(self, model, step, d):
        info = convert.expert_parallel_info(model)
        if info is not None:
            # Experts are sliced over the ep group: the ranks of the master's group gather them one decoder
            # layer at a time (a collective among them), the master then broadcasts the full layer.
            if not info["writer"]:
                return
            per_layer = _gathered_layers(model, info)
            n_groups = len(layer_groups([k for k in model.state_dict() if "lora_" not in k]))
        else:
            if not self.world.is_master:
                return
            full = convert.model_state(model, "hf")
            per_layer = [{n: full[n] for n in names} for names in layer_groups(list(full))]
            n_groups = len(per_layer)            # what the receiver is told to expect is what is sent
            info = None
        device = next(model.parameters()).device
        if self.world.is_master:
            self._connect(device)
            _broadcast(self.pg, torch.tensor([n_groups], dtype=torch.int64, device=device))
        for sd in per_layer:
            if not self.world.is_master:
                continue
            names = list(sd)
            meta = [(n, tuple(sd[n].shape), str(sd[n].dtype).replace("torch.", "")) for n in names]
            blob = torch.frombuffer(bytearray(pickle.dumps(meta)), dtype=torch.uint8).to(device)
            size = torch.tensor([blob.numel()], dtype=torch.int64, device=device)
            _broadcast(self.pg, size)
            _broadcast(self.pg, blob)
            by_dtype: dict[str, list[torch.Tensor]] = {}
            for n, _, dt in meta:
                by_dtype.setdefault(dt, []).append(sd[n].detach().reshape(-1))
            for dt in sorted(by_dtype):
                _broadcast(self.pg, torch.cat(by_dtype[dt]))


def _gathered_layers(model, info):
    """Yields the HF-layout tensors of one decoder layer at a time (then of everything else) with the
    expert stacks all-gathered over the ep group, so that at most one layer's experts are held twice."""
    native = {k: v for k, v in model.state_dict().items() if "lora_" not in k}
    for names in layer_groups(list(native)):
        part = {n: (convert.gather_expert_shards(native[n], info) if convert.is_expert_sharded_key(n) else native[n])
                for n in names}
        yield convert.native_to_hf(part, model.arch)


class NCCLWeightReceiver:
    """Engine-side worker: joins the group as rank ``rank`` and applies broadcast layers."""

    def __init__(self, host: str, port: int, rank: int, world_size: int, timeout: int = 1200):
        self.host, self.port, self.rank, self.world_size, self.timeout = host, port, rank, world_size, timeout
        self.pg = None

    def connect(self, device: torch.device | None = None) -> None:
        device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                            else torch.device("cpu"))
        self.device = device
        self.pg, self.store = _new_group(self.host, self.port, self.rank, self.world_size, self.timeout, device)

    @torch.no_grad()
    def receive_into(self, engine) -> None:
        model, dev = engine.model, self.device
        header = torch.zeros(1, dtype=torch.int64, device=dev)
        _broadcast(self.pg, header)
        for _ in range(int(header.item())):
            size = torch.zeros(1, dtype=torch.int64, device=dev)
            _broadcast(self.pg, size)
            blob = torch.empty(int(size.item()), dtype=torch.uint8, device=dev)
            _broadcast(self.pg, blob)
            meta = pickle.loads(bytes(blob.cpu().numpy()))
            by_dtype: dict[str, list] = {}
            for n, shape, dt in meta:
                by_dtype.setdefault(dt, []).append((n, shape))
            sd = {}
            for dt in sorted(by_dtype):
                total = sum(int(torch.Size(s).numel()) for _, s in by_dtype[dt])
                flat = torch.empty(total, dtype=getattr(torch, dt), device=dev)
                _broadcast(self.pg, flat)
                off = 0
                for n, shape in by_dtype[dt]:
                    k = int(torch.Size(shape).numel())
                    sd[n] = flat[off:off + k].view(shape)
                    off += k
            convert.load_model_state(model, sd, "hf", strict=False)
        engine.cache.blocks.clear_prefix_cache()
        engine.policy_version += 1
