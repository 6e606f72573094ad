"""Rollout engine: continuous batching over the paged KV cache.

One background thread runs the step loop (prefill of admitted requests, then one decode step
for every running sequence); requests arrive from the HTTP server's event loop. Pausing
freezes in-flight requests without aborting them (the reference pauses vLLM with
``mode="keep", clear_cache=False``; src/prime_rl/inference/vllm/server.py:66-76); weight
updates happen only while paused.
"""

from __future__ import annotations

import asyncio
import threading
import time
import uuid
from dataclasses import dataclass, field

import torch

from ..utils.logger import get_logger
from .kv_cache import KVCache, OutOfPages, SequenceKV
from .runner import ModelRunner, StepInput
from .sampler import SamplingParams, sample


@dataclass
class Request:
    prompt: list[int]
    params: SamplingParams
    cache_salt: str = ""
    request_id: str = field(default_factory=lambda: uuid.uuid4().hex)
    # state
    kv: SequenceKV = field(default_factory=SequenceKV)
    output: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    prompt_logprobs: list[float] | None = None
    routed: list[torch.Tensor] = field(default_factory=list)
    masks: list[torch.Tensor] = field(default_factory=list)
    finish_reason: str | None = None
    arrival: float = field(default_factory=time.monotonic)
    future: asyncio.Future | None = None
    loop: asyncio.AbstractEventLoop | None = None
    generator: torch.Generator | None = None
    prefilled: bool = False
    preemptions: int = 0
    swapped: object = None          # kv_cache.HostKV while the request waits with its K / V in host memory
    # prefill / decode disaggregation: a prefill-only request ends after its first sampled token with its K / V
    # moved to host memory (``handoff``), ready to be imported by another engine (``Engine.submit_prefilled``)
    prefill_only: bool = False
    handoff: object = None
    # image inputs: {"pixel_values": [patches, patch_dim], "image_grid_thw": [images, 3]}; ``mm_state`` is what the
    # first prefill step derives from them (features per prompt token, 3-axis positions, position shift of the
    # generated tokens)
    mm: dict | None = None
    mm_state: dict | None = None

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt + self.output


class Engine:
    def __init__(self, model, *, num_pages: int = 4096, page_size: int = 16, max_running: int = 256,
                 max_prefill_tokens: int = 16384, eos_token_id: int | None = None, enable_prefix_cache: bool = True,
                 use_cuda_graphs: bool = False, max_model_len: int = 8192, weight_dtype: str = "bf16", tp=None,
                 keep_bf16_weights: bool = True, kv_offload_bytes: int = 0, expert_parallel: bool = False,
                 vision=None, image_token_id: int | None = None, mrope_section: tuple[int, int, int] = (11, 11, 10)):
        """``expert_parallel`` (with ``tp``): the ranks split the experts by index instead of by width
        (``engine/tp.py``). ``kv_offload_bytes`` > 0: a request that is preempted for lack of pages keeps its K / V in (pinned) host
        memory up to that many bytes in total and resumes without a second prefill (the reference configures this
        as ``kv_cache_offload.cpu.num_bytes`` of its serving stack,
        packages/prime-rl-configs/src/prime_rl/configs/inference.py:216-300)."""
        arch = model.arch
        self.kv_offload_bytes, self.kv_offloaded = int(kv_offload_bytes), 0
        self.model = model.eval()
        self.weight_dtype = weight_dtype
        # tensor parallelism (engine/tp.py): this process holds one shard and steps in lockstep with its peers
        self.tp = tp
        self.tp_size = tp.size if tp is not None else 1
        self._inbox: list[Request] = []
        self._commands: list[tuple] = []
        self.mark = None
        self._sampling_cache = None
        if tp is not None and tp.size > 1:
            from .tp import shard_model_

            if getattr(model, "tp_size", 1) != tp.size:
                shard_model_(self.model, tp.rank, tp.size, expert_parallel=expert_parallel)
            if tp.max_tokens < max(max_prefill_tokens, max_model_len):
                raise ValueError("the tensor-parallel buffers are smaller than the largest step the engine may run")
        # fp8 serving: with ``keep_bf16_weights=False`` the bf16 storage of every quantised projection is
        # released (weight updates are then quantised tensor by tensor as they arrive)
        self.drop_bf16 = weight_dtype == "fp8" and not keep_bf16_weights
        if weight_dtype == "fp8":
            from ..models.model import quantize_fp8_

            quantize_fp8_(self.model, drop_bf16=self.drop_bf16)
        p = next(p for p in model.parameters() if p.numel() > 0)
        self.device = p.device
        self.cache = KVCache(arch.num_hidden_layers, num_pages, page_size, arch.num_key_value_heads // self.tp_size,
                             arch.head_dim, p.dtype, p.device)
        from .hybrid import HybridRunner, needs_hybrid_runner

        if needs_hybrid_runner(model):
            # layers with a recurrent state (Mamba-2, gated delta-net): the state of a prefix cannot be shared through
            # the page cache and is not part of a host-memory swap, so both are off for these families
            if self.tp_size > 1:
                raise NotImplementedError("tensor parallelism of the rollout engine covers the attention decoder families")
            enable_prefix_cache, self.kv_offload_bytes = False, 0
            self.runner = HybridRunner(model, self.cache, max_model_len=max_model_len)
        else:
            self.runner = ModelRunner(model, self.cache, use_cuda_graphs=use_cuda_graphs, max_model_len=max_model_len,
                                      tp=tp if self.tp_size > 1 else None, shared_prefix_decode=enable_prefix_cache)
        self.max_running, self.max_prefill_tokens = max_running, max_prefill_tokens
        self.eos, self.enable_prefix_cache = eos_token_id, enable_prefix_cache
        self._hybrid = isinstance(self.runner, HybridRunner)
        # image inputs (``models/vision.py: VisionTower``): features replace the embeddings of the placeholder tokens
        self.vision, self.image_token_id = vision, image_token_id
        if vision is not None:
            if not isinstance(self.runner, HybridRunner):
                raise NotImplementedError("image inputs are served for the families of the recurrent-state runner")
            self.runner.mrope_section = tuple(mrope_section)
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.lock = threading.Lock()
        self.wake = threading.Condition(self.lock)
        self.paused = False
        self.idle_paused = threading.Event()
        self.stop_flag = False
        self.thread: threading.Thread | None = None
        self.logger = get_logger()
        self.policy_version = 0
        self.weight_receiver = None          # in-memory weight transport endpoint (NCCL receiver or peer-memory port)
        self.stats = dict(prompt_tokens=0, generation_tokens=0, preemptions=0, prefix_hits=0, prefix_queries=0,
                          requests=0, steps=0)
        self.last_step_time = time.monotonic()

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "Engine":
        if self.thread is None:
            self.thread = threading.Thread(target=self._loop, name="engine-loop", daemon=True)
            self.thread.start()
        return self

    def shutdown(self) -> None:
        with self.wake:
            self.stop_flag = True
            self.wake.notify_all()
        if self.thread is not None:
            self.thread.join(timeout=10)
        if self.tp_size > 1 and self.tp.rank == 0:          # release the other ranks from their follow() loops
            with self.lock:
                self._commands.append(("stop",))
            self._tp_sync()

    def pause(self, timeout: float = 60.0) -> None:
        """Returns once the step loop is parked (no kernel of a step in flight)."""
        with self.wake:
            self.paused = True
            self.idle_paused.clear()
            self.wake.notify_all()
        if self.thread is not None and not self.idle_paused.wait(timeout):
            raise TimeoutError("engine did not pause in time")

    def resume(self) -> None:
        with self.wake:
            self.paused = False
            self.wake.notify_all()

    def is_alive(self) -> bool:
        return self.thread is not None and self.thread.is_alive()

    # ------------------------------------------------------------------ requests
    def submit(self, req: Request) -> Request:
        if req.params.seed is not None:
            req.generator = torch.Generator(device=self.device).manual_seed(req.params.seed)
        with self.wake:
            # with tensor parallelism a request enters the queue when rank 0 announces it to all ranks
            (self._inbox if self.tp_size > 1 else self.waiting).append(req)
            self.stats["requests"] += 1
            self.wake.notify_all()
        return req

    # ------------------------------------------------------------------ tensor-parallel lockstep
    def _tp_sync(self) -> bool:
        """Rank 0 announces the requests and admin commands that arrived since the last step; every rank
        queues / runs them in the same order. Returns False once a stop command came through."""
        tp = self.tp
        msg = None
        if tp.rank == 0:
            with self.lock:
                new, self._inbox = self._inbox, []
                cmds, self._commands = self._commands, []
            msg = {"new": [(r.prompt, r.params, r.cache_salt) for r in new], "cmds": cmds}
        msg = tp.broadcast_control(msg)
        if tp.rank != 0:
            new = [Request(prompt=list(p), params=params, cache_salt=salt) for p, params, salt in msg["new"]]
            for r in new:
                if r.params.seed is not None:
                    r.generator = torch.Generator(device=self.device).manual_seed(r.params.seed)
        with self.lock:
            self.waiting.extend(new)
        alive = True
        for cmd in msg["cmds"]:
            if cmd[0] == "update_weights":
                self._update_weights_local(cmd[1])
            elif cmd[0] == "mark":                  # a label every rank sees at the same step (benchmarks)
                self.mark = cmd[1]
            elif cmd[0] == "clear_prefix_cache":
                self.cache.blocks.clear_prefix_cache()
            elif cmd[0] == "init_broadcaster":
                self._init_broadcaster_local(cmd[1])
            elif cmd[0] == "receive_weights":
                self.weight_receiver.receive_into(self)
            elif cmd[0] == "stop":
                alive = False
        return alive

    def follow(self) -> None:
        """Step loop of the ranks other than 0: wait for rank 0's announcement, then take the same step."""
        assert self.tp is not None and self.tp.rank != 0
        while self._tp_sync():
            if self.waiting or self.running:
                self._step_local()

    async def generate(self, prompt: list[int], params: SamplingParams, cache_salt: str = "",
                       mm: dict | None = None) -> Request:
        """``mm``: image inputs of the prompt (``pixel_values``, ``image_grid_thw``), whose features take the place of
        the embeddings of the placeholder tokens."""
        loop = asyncio.get_running_loop()
        req = Request(prompt=list(prompt), params=params, cache_salt=cache_salt, loop=loop,
                      future=loop.create_future(), mm=mm)
        self.submit(req)
        return await req.future

    # ------------------------------------------------------------------ prefill / decode disaggregation
    def _check_handoff_supported(self) -> None:
        from .hybrid import HybridRunner

        if isinstance(self.runner, HybridRunner) or self.tp_size > 1:
            raise NotImplementedError("K / V hand-off between engines covers single-process engines of the attention "
                                      "decoder families (a recurrent state or a sharded cache is not exported)")

    async def prefill(self, prompt: list[int], params: SamplingParams, cache_salt: str = "") -> Request:
        """Prefill role: runs the prompt, samples the first token and returns with ``handoff`` = the K / V of the
        prompt in host memory (``finish_reason == "prefill_done"``; a request that ends at its first token
        finishes normally and has nothing to hand off)."""
        self._check_handoff_supported()
        loop = asyncio.get_running_loop()
        req = Request(prompt=list(prompt), params=params, cache_salt=cache_salt, loop=loop,
                      future=loop.create_future(), prefill_only=True)
        self.submit(req)
        return await req.future

    def submit_prefilled(self, prompt: list[int], output: list[int], logprobs: list[float], host_kv,
                         params: SamplingParams, cache_salt: str = "", loop=None, future=None) -> Request:
        """Decode role: a request whose prompt was run by another engine. ``host_kv`` (``kv_cache.HostKV``) holds the
        K / V of the prompt; the request joins the queue like one that was swapped out and continues from
        ``output[-1]`` without a prefill step."""
        self._check_handoff_supported()
        lay = self.cache.k.shape
        if tuple(host_kv.data.shape[1:2]) != (lay[0],) or tuple(host_kv.data.shape[3:]) != tuple(lay[2:]):
            raise ValueError(f"imported K / V {tuple(host_kv.data.shape)} does not fit this engine's cache layout "
                             f"{tuple(lay)} (layers, page size, kv heads and head dim must match)")
        req = Request(prompt=list(prompt), params=params, cache_salt=cache_salt, loop=loop, future=future)
        req.output, req.logprobs = list(output), list(logprobs)
        req.swapped, req.prefilled = host_kv, True
        self.kv_offloaded += host_kv.nbytes
        self.stats["kv_imports"] = self.stats.get("kv_imports", 0) + 1
        return self.submit(req)

    def generate_sync(self, prompts: list[list[int]], params: SamplingParams, cache_salt: str = "") -> list[Request]:
        """Blocking helper for tests and benchmarks (runs the loop inline if no thread is active)."""
        reqs = [self.submit(Request(prompt=list(p), params=params, cache_salt=cache_salt)) for p in prompts]
        if self.thread is None:
            while any(r.finish_reason is None for r in reqs):
                self.step()
        else:
            while any(r.finish_reason is None for r in reqs):
                time.sleep(0.001)
        return reqs

    # ------------------------------------------------------------------ step loop
    def _loop(self) -> None:
        while True:
            with self.wake:
                while not self.stop_flag and (self.paused or not (self.waiting or self.running or self._inbox
                                                                  or self._commands)):
                    if self.paused:
                        self.idle_paused.set()
                    self.wake.wait(timeout=0.5)
                if self.stop_flag:
                    return
            try:
                self.step()
            except Exception as e:  # fail the in-flight requests, keep serving
                self.logger.exception(f"engine step failed: {e}")
                with self.lock:
                    doomed, self.running = self.running, []
                for r in doomed:
                    self._finish(r, "error")

    def _finish(self, r: Request, reason: str) -> None:
        r.finish_reason = reason
        if reason == "prefill_done" and r.kv.pages:
            r.handoff = self.cache.swap_out(r.kv, pin=False)       # the pages return to the pool
        self.cache.free(r.kv)
        if r.swapped is not None:
            self.kv_offloaded -= r.swapped.nbytes
            r.swapped = None
        if r.future is not None and r.loop is not None:
            try:
                r.loop.call_soon_threadsafe(lambda: r.future.done() or r.future.set_result(r))
            except RuntimeError:
                pass  # the client's event loop is gone (caller shut down mid-request)

    def _admit(self) -> list[Request]:
        """Moves waiting requests to running while pages and the prefill budget allow."""
        admitted, budget = [], self.max_prefill_tokens
        seen: set = set()
        with self.lock:
            while self.waiting and len(self.running) + len(admitted) < self.max_running:
                r = self.waiting[0]
                if r.swapped is not None:
                    # K / V waits in host memory: bring it back instead of prefilling again
                    need = r.swapped.data.shape[2] + 1
                    if self.cache.blocks.num_available < need and (self.running or admitted):
                        break
                    self.waiting.pop(0)
                    self.cache.swap_in(r.kv, r.swapped)
                    self.kv_offloaded -= r.swapped.nbytes
                    r.swapped = None
                    self.stats["kv_swap_ins"] = self.stats.get("kv_swap_ins", 0) + 1
                    self.running.append(r)
                    continue
                toks = r.all_tokens
                need_pages = (len(toks) + self.cache.page_size) // self.cache.page_size + 1
                cost = len(toks)
                if self._hybrid and r.mm is None and not r.params.prompt_logprobs:
                    # a further sample of a prompt admitted in this round forks the first one's prefill: it costs no
                    # prompt tokens and, until it diverges, one page of its own
                    key = (r.cache_salt, tuple(toks))
                    if key in seen:
                        cost, need_pages = 0, 2
                    seen.add(key)
                if cost > budget and admitted:
                    break
                if self.cache.blocks.num_available < need_pages and (self.running or admitted):
                    break
                self.waiting.pop(0)
                admitted.append(r)
                budget -= cost
        return admitted

    def _preempt_one(self) -> bool:
        """Out of pages: push the most recent running request back to the queue (its KV is
        recomputed on re-admission)."""
        with self.lock:
            if len(self.running) <= 1:
                return False
            r = self.running.pop()
            nbytes = 2 * len(r.kv.pages) * self.cache.k[:, 0].numel() * self.cache.k.element_size()
            if (self.kv_offload_bytes and r.prefilled and r.kv.pages
                    and self.kv_offloaded + nbytes <= self.kv_offload_bytes):
                r.swapped = self.cache.swap_out(r.kv)          # resumes where it stopped
                self.kv_offloaded += nbytes
                self.stats["kv_swap_outs"] = self.stats.get("kv_swap_outs", 0) + 1
            else:
                self.cache.free(r.kv)
                r.prefilled = False
            r.preemptions += 1
            self.stats["preemptions"] += 1
            self.waiting.insert(0, r)
        return True

    def step(self) -> None:
        if self.tp_size > 1:
            if not self._tp_sync():
                return
            if not (self.waiting or self.running):
                return
        self._step_local()

    def _step_local(self) -> None:
        self.stats["steps"] += 1
        self.last_step_time = time.monotonic()
        new = self._admit()
        if new:
            self._prefill(new)
        with self.lock:
            batch = [r for r in self.running if r.prefilled and r.finish_reason is None]
        if batch:
            self._decode(batch)
        if self.tp_size > 1 and self.device.type == "cuda":
            # a reduce whose bounded wait ran out (a peer that left) wrote nothing: fail the step, not the tokens
            from ..ops import _runtime as rt

            rt.check_status(self.device)

    # ------------------------------------------------------------------ prefill
    def _prefill(self, reqs: list[Request]) -> None:
        followers: list[tuple[Request, Request]] = []
        all_reqs = reqs
        if self._hybrid and len(reqs) > 1:
            # samples of one prompt (a group of the RL algorithm arrives together): the families of this runner have
            # no page-level prefix cache, so the prompt is run once and the other samples fork pages and states
            first: dict = {}
            keep = []
            for r in reqs:
                key = (r.cache_salt, tuple(r.all_tokens)) if (r.mm is None and not r.params.prompt_logprobs
                                                              and r.kv.length == 0) else id(r)
                if key in first:
                    followers.append((r, first[key]))
                else:
                    first[key] = r
                    keep.append(r)
            reqs = keep
        inputs = []
        for r in reqs:
            toks = r.all_tokens
            self.stats["prefix_queries"] += len(toks)
            if self.enable_prefix_cache and not r.params.prompt_logprobs and r.mm is None:
                pages = self.cache.blocks.lookup_prefix(r.cache_salt, toks[:-1])
                r.kv.pages, r.kv.length = pages, len(pages) * self.cache.page_size
                self.stats["prefix_hits"] += r.kv.length
            inp = StepInput(r.kv, toks[r.kv.length:], want_all_logits=r.params.prompt_logprobs)
            if r.mm is not None:
                self._attach_image_inputs(r, inp, r.kv.length, len(toks))
            inputs.append(inp)
        try:
            logits, offsets = self.runner.forward(inputs)
        except OutOfPages:
            for r in reqs:
                self.cache.free(r.kv)
            with self.lock:
                self.waiting = all_reqs + self.waiting
            if not self._preempt_one():
                raise
            return
        self.stats["prompt_tokens"] += sum(len(i.tokens) for i in inputs)
        rows = []
        for r, inp, off in zip(reqs, inputs, offsets):
            n = len(inp.tokens)
            if r.params.prompt_logprobs:
                lp = torch.log_softmax(logits[off:off + n - 1], -1)
                tgt = torch.tensor(r.prompt[1:], device=lp.device)
                r.prompt_logprobs = [0.0] + lp.gather(1, tgt[:n - 1, None]).squeeze(1).tolist()
                rows.append(off + n - 1)
            else:
                rows.append(off)
            if self.enable_prefix_cache and r.mm is None:
                self.cache.blocks.register_prefix(r.cache_salt, r.all_tokens, r.kv.pages)
            r.prefilled = True
        routed_rows = [sum(len(i.tokens) for i in inputs[:j + 1]) - 1 for j in range(len(inputs))]
        if followers:
            row_of = {id(r): (rows[j], routed_rows[j]) for j, r in enumerate(reqs)}
            for f, leader in followers:
                f.kv = self.cache.fork(leader.kv)
                self.runner.fork_state(leader.kv, f.kv)
                f.prefilled = True
                rows.append(row_of[id(leader)][0])
                routed_rows.append(row_of[id(leader)][1])
                reqs.append(f)
            self.stats["prefill_forks"] = self.stats.get("prefill_forks", 0) + len(followers)
        self._sample_and_append(reqs, logits[torch.tensor(rows, device=logits.device)], self.runner.last_routed,
                                routed_rows)
        with self.lock:
            self.running.extend(r for r in reqs if r.finish_reason is None)

    # ------------------------------------------------------------------ decode
    def _attach_image_inputs(self, r: Request, inp: StepInput, start: int, end: int) -> None:
        """Image features and 3-axis positions of tokens ``[start, end)`` of ``r`` (prompt + output so far)."""
        if self.vision is None:
            raise ValueError("this engine was started without a vision tower")
        st = r.mm_state
        if st is None:
            from ..models.vision import mrope_position_ids

            ids = torch.tensor(r.prompt)
            is_image = ids == self.image_token_id
            with torch.no_grad():
                feats = self.vision(r.mm["pixel_values"].to(self.device), r.mm["image_grid_thw"].to(self.device))
            if int(is_image.sum()) != feats.shape[0]:
                raise ValueError(f"{int(is_image.sum())} image tokens but {feats.shape[0]} image features")
            embeds = torch.zeros(len(r.prompt), feats.shape[1], dtype=feats.dtype, device=feats.device)
            embeds[is_image.to(feats.device)] = feats
            pos3 = mrope_position_ids(is_image.long(), [len(r.prompt)], r.mm["image_grid_thw"].tolist(),
                                      self.vision.config.spatial_merge_size)
            st = r.mm_state = {"embeds": embeds, "is_image": is_image, "pos3": pos3,
                               "delta": int(pos3.max()) + 1 - len(r.prompt)}
        P = len(r.prompt)
        pos = torch.arange(start, end)
        pos3 = (pos + st["delta"]).unsqueeze(0).repeat(3, 1)
        if start < P:
            hi = min(end, P)
            pos3[:, : hi - start] = st["pos3"][:, start:hi]
            rows = torch.zeros(end - start, dtype=torch.bool)
            rows[: hi - start] = st["is_image"][start:hi]
            emb = torch.zeros(end - start, st["embeds"].shape[1], dtype=st["embeds"].dtype, device=st["embeds"].device)
            emb[: hi - start] = st["embeds"][start:hi]
            inp.embeds, inp.embed_rows = emb, rows
        inp.pos3 = pos3

    def _decode(self, reqs: list[Request]) -> None:
        inputs = [StepInput(r.kv, [r.output[-1]]) for r in reqs]
        for r, inp in zip(reqs, inputs):
            if r.mm is not None:
                self._attach_image_inputs(r, inp, r.kv.length, r.kv.length + 1)
        while True:
            try:
                logits, _ = self.runner.forward(inputs)
                break
            except OutOfPages:
                if not self._preempt_one():
                    raise
                with self.lock:
                    alive = set(id(r) for r in self.running)
                keep = [(r, i) for r, i in zip(reqs, inputs) if id(r) in alive]
                reqs, inputs = [k[0] for k in keep], [k[1] for k in keep]
                if not reqs:
                    return
        self._sample_and_append(reqs, logits, self.runner.last_routed, list(range(len(reqs))))
        with self.lock:
            self.running = [r for r in self.running if r.finish_reason is None]

    def _sample_and_append(self, reqs, logits, routed, routed_rows) -> None:
        dev = logits.device
        # the sampling parameters of an unchanged set of requests stay on the device from step to step
        c = self._sampling_cache           # holds the request objects themselves, so an identity match cannot be stale
        if c is None or len(c[0]) != len(reqs) or any(a is not b for a, b in zip(c[0], reqs)):
            self._sampling_cache = (list(reqs),
                                    torch.tensor([r.params.temperature for r in reqs], dtype=torch.float32, device=dev),
                                    torch.tensor([r.params.top_k for r in reqs], dtype=torch.long, device=dev),
                                    torch.tensor([r.params.top_p for r in reqs], dtype=torch.float32, device=dev))
        _, temp, top_k, top_p = self._sampling_cache
        want_mask = any(r.params.return_sampling_mask and r.params.truncated for r in reqs)
        gen = reqs[0].generator if len(reqs) == 1 else None
        tok, lp, masks = sample(logits, temp, top_k, top_p, generator=gen, want_mask=want_mask,
                                truncated=any(r.params.truncated for r in reqs))
        if self.tp_size > 1:                       # every rank appends rank 0's draw
            tok, lp = self.tp.broadcast_sample(tok, lp)
        both = torch.stack([tok.double(), lp.double()]).tolist()       # one device-to-host read per step
        tok_l, lp_l = [int(t) for t in both[0]], both[1]
        self.stats["generation_tokens"] += len(reqs)
        for i, r in enumerate(reqs):
            r.output.append(tok_l[i])
            r.logprobs.append(lp_l[i])
            if routed is not None and r.params.return_routed_experts:
                r.routed.append(routed[routed_rows[i]].to("cpu", torch.int16))
            if masks is not None and r.params.return_sampling_mask:
                r.masks.append(masks[i].cpu())
            n = len(r.output)
            if r.prefill_only and n >= 1 and n < r.params.max_tokens and not \
                    (n >= r.params.min_tokens and (tok_l[i] == self.eos or tok_l[i] in r.params.stop_token_ids)):
                self._finish(r, "prefill_done")
            elif n >= r.params.max_tokens:
                self._finish(r, "length")
            elif n >= r.params.min_tokens and (tok_l[i] == self.eos or tok_l[i] in r.params.stop_token_ids):
                self._finish(r, "stop")

    # ------------------------------------------------------------------ weights
    def update_weights_from_dir(self, weight_dir: str) -> None:
        """Must be called while paused. HF safetensors directory, or a PEFT adapter directory."""
        from pathlib import Path

        from ..trainer.weights import load_hf_checkpoint

        assert self.paused or self.thread is None, "update_weights requires a paused engine"
        if self.tp_size > 1:
            # the step loop is parked, so this thread owns the control channel: all ranks load their shards
            assert self.tp.rank == 0, "weight updates enter through rank 0"
            with self.lock:
                self._commands.append(("update_weights", str(weight_dir)))
            self._tp_sync()
            return
        self._update_weights_local(weight_dir)

    def _update_weights_local(self, weight_dir: str) -> None:
        from pathlib import Path

        from ..trainer.weights import load_hf_checkpoint

        load_hf_checkpoint(self.model, Path(weight_dir), strict=False)
        if self.weight_dtype == "fp8":
            from ..models.model import quantize_fp8_

            quantize_fp8_(self.model, drop_bf16=self.drop_bf16)
        self.cache.blocks.clear_prefix_cache()
        self.policy_version += 1

    # ------------------------------------------------------------------ in-memory weight updates
    def init_broadcaster(self, spec: dict) -> None:
        """Joins the trainer's in-memory weight transport. ``spec`` is the body of ``/init_broadcaster``:
        ``type`` ("nccl" | "p2p"), ``rank_offset`` (index of this engine among all engine GPUs) and the
        transport's own fields. With tensor parallelism every rank of the engine joins: rank r takes
        transport slot ``rank_offset + r`` and, on every update, keeps its own slices of what arrives."""
        if self.tp_size > 1:
            assert self.tp.rank == 0, "admin commands enter through rank 0"
            with self.lock:
                self._commands.append(("init_broadcaster", dict(spec)))
            self._tp_sync()
            return
        self._init_broadcaster_local(spec)

    def _init_broadcaster_local(self, spec: dict) -> None:
        from pathlib import Path

        slot = int(spec.get("rank_offset", 0)) + (self.tp.rank if self.tp_size > 1 else 0)
        if spec.get("type") == "p2p":
            from ..transports.weights.p2p import P2PWeightPort

            tp = (self.tp.rank, self.tp_size, bool(getattr(self.model, "tp_expert_parallel", False))) \
                if self.tp_size > 1 else None
            self.weight_receiver = P2PWeightPort(self.model, Path(spec["run_dir"]), slot, spec.get("quantize"), tp=tp)
            return
        from ..transports.weights.nccl import NCCLWeightReceiver

        self.weight_receiver = NCCLWeightReceiver(host=spec["host"], port=int(spec["port"]), rank=slot + 1,
                                                  world_size=int(spec["inference_world_size"]) + 1,
                                                  timeout=int(spec.get("timeout", 1200)))
        self.weight_receiver.connect(self.device if self.device.type == "cuda" else None)

    def receive_weights(self) -> None:
        """Takes part in one in-memory weight update (engine paused). Tensor-parallel engines: all ranks."""
        if self.weight_receiver is None:
            raise RuntimeError("no in-memory broadcaster was initialised")
        assert self.paused or self.thread is None, "weight updates require a paused engine"
        if self.tp_size > 1:
            assert self.tp.rank == 0
            with self.lock:
                self._commands.append(("receive_weights",))
            self._tp_sync()
            return
        self.weight_receiver.receive_into(self)

    def clear_prefix_cache(self) -> None:
        """Drops every cached prefix (their pages return to the free list once no running request uses them).
        With tensor parallelism the command travels with the next step announcement so that every rank drops
        the same pages at the same step."""
        if self.tp_size > 1:
            with self.lock:
                self._commands.append(("clear_prefix_cache",))
        else:
            self.cache.blocks.clear_prefix_cache()

    def metrics(self) -> dict:
        with self.lock:
            return dict(self.stats, running=len(self.running), waiting=len(self.waiting),
                        kv_usage=self.cache.blocks.usage, policy_version=self.policy_version)
