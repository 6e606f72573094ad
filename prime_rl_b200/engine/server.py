"""HTTP surface of the rollout engine (FastAPI).

Routes (same paths and payloads as the reference's vLLM wrapper,
src/prime_rl/inference/vllm/server.py:66-147 and serving_tokens.py:46-116):

  POST /inference/v1/generate   token-in / token-out with logprobs, routed experts, sampling mask
  POST /v1/chat/completions, /v1/completions   OpenAI-style (needs a tokenizer)
  GET  /v1/models, /health, /liveness, /metrics
  POST /pause, /resume, /update_weights, /init_broadcaster, /load_lora_adapter
"""

from __future__ import annotations

import asyncio
import base64
import time
from pathlib import Path

import numpy as np
import torch
from fastapi import FastAPI, HTTPException, Request as HTTPRequest
from fastapi.responses import JSONResponse, PlainTextResponse

from .engine import Engine
from .sampler import SamplingParams


def _encode_routed(routed: list[torch.Tensor], start: int = 0) -> dict | None:
    if not routed:
        return None
    arr = torch.stack(routed).numpy().astype(np.int16)        # [tokens, layers, topk]
    return {"data": base64.b64encode(arr.tobytes()).decode(), "shape": list(arr.shape), "start": start,
            "dtype": "int16"}


def _decode_images(mm: dict | None) -> dict | None:
    """``multi_modal_data`` of a generate request: ``pixel_values`` as ``{"dtype", "shape", "data"}`` with base64 bytes (the
    layout of the trainer's wire tensors) or as nested lists, ``image_grid_thw`` as ``[[t, h, w], ...]``."""
    if not mm:
        return None
    import base64

    pv = mm.get("pixel_values")
    if pv is None or mm.get("image_grid_thw") is None:
        raise HTTPException(400, "multi_modal_data needs pixel_values and image_grid_thw")
    if isinstance(pv, dict):
        raw = base64.b64decode(pv["data"])
        pixels = torch.frombuffer(bytearray(raw), dtype=getattr(torch, pv["dtype"])).reshape(pv["shape"]).clone()
    else:
        pixels = torch.tensor(pv, dtype=torch.float32)
    return {"pixel_values": pixels, "image_grid_thw": torch.tensor(mm["image_grid_thw"], dtype=torch.long)}


def _encode_mask(masks: list[torch.Tensor]) -> dict | None:
    if not masks:
        return None
    counts = np.array([m.numel() for m in masks], dtype=np.int32)
    ids = np.concatenate([m.numpy().astype(np.int32) for m in masks]) if counts.sum() else np.zeros(0, np.int32)
    return {"ids": base64.b64encode(ids.tobytes()).decode(), "counts": base64.b64encode(counts.tobytes()).decode()}


def build_app(engine: Engine, model_name: str, tokenizer=None, liveness_timeout: float = 30.0,
              weight_receiver=None) -> FastAPI:
    app = FastAPI(title="prime-rl-b200 inference")
    app.state.engine = engine
    if weight_receiver is not None:
        engine.weight_receiver = weight_receiver

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/liveness")
    async def liveness():
        # the step loop must have made progress (or be idle / paused) within the timeout
        age = time.monotonic() - engine.last_step_time
        busy = bool(engine.running or engine.waiting)
        if not engine.is_alive() or (busy and not engine.paused and age > liveness_timeout):
            return JSONResponse({"status": "engine_unresponsive"}, status_code=503)
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "prime-rl-b200"}]}

    @app.get("/metrics")
    async def metrics():
        m = engine.metrics()
        hit = m["prefix_hits"]
        lines = [
            f"vllm:num_requests_running {m['running']}", f"vllm:num_requests_waiting {m['waiting']}",
            f"vllm:kv_cache_usage_perc {m['kv_usage']:.6f}", f"vllm:gpu_cache_usage_perc {m['kv_usage']:.6f}",
            f"vllm:num_preemptions_total {m['preemptions']}", f"vllm:prompt_tokens_total {m['prompt_tokens']}",
            f"vllm:generation_tokens_total {m['generation_tokens']}", f"vllm:prefix_cache_hits_total {hit}",
            f"vllm:prefix_cache_queries_total {m['prefix_queries']}", f"vllm:request_success_total {m['requests']}",
            f"prime_rl:policy_version {m['policy_version']}",
        ]
        # counters that exist once the engine has used the path: K / V swaps of preempted requests, imports from a
        # prefill engine, prompts shared by forking in the recurrent-state runner
        for key in ("kv_swap_outs", "kv_swap_ins", "kv_imports", "prefill_forks"):
            if key in m:
                lines.append(f"prime_rl:{key}_total {m[key]}")
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/inference/v1/generate")
    async def generate(body: dict):
        token_ids = body.get("token_ids")
        if not token_ids:
            raise HTTPException(400, "token_ids is required")
        sp = dict(body.get("sampling_params") or {})
        n = int(sp.pop("n", 1) or 1)
        if engine.runner.capture_routed:
            sp.setdefault("return_routed_experts", True)
        params = SamplingParams.from_dict(sp)
        if body.get("return_sampling_mask") or app.state.__dict__.get("return_sampling_mask"):
            params.return_sampling_mask = True
        salt = str(body.get("cache_salt", ""))
        kvp = body.get("kv_transfer_params")
        if kvp:
            # decode role of a disaggregated deployment: the prompt was run by a prefill engine, whose K / V and first
            # token come with the request (``/inference/v1/prefill`` of that engine produced them)
            from .kv_cache import HostKV

            first = body.get("prefill_output") or {}
            loop = asyncio.get_running_loop()
            fut = loop.create_future()
            try:
                engine.submit_prefilled(token_ids, list(first.get("token_ids") or []), list(first.get("logprobs") or []),
                                        HostKV.from_file(kvp), params, salt, loop=loop, future=fut)
            except (ValueError, NotImplementedError, OSError) as e:
                raise HTTPException(400, f"cannot import the transferred K / V: {e}")
            reqs = [await fut]
        else:
            mm = _decode_images(body.get("multi_modal_data"))
            reqs = await asyncio.gather(*[engine.generate(token_ids, params, salt, mm=mm) for _ in range(n)])
        choices = []
        for i, r in enumerate(reqs):
            choices.append({
                "index": i, "token_ids": r.output, "logprobs": r.logprobs, "finish_reason": r.finish_reason,
                "prompt_logprobs": r.prompt_logprobs, "routed_experts": _encode_routed(r.routed),
                "sampling_mask": _encode_mask(r.masks)})
        return {"id": reqs[0].request_id, "model": body.get("model", model_name), "choices": choices,
                "usage": {"prompt_tokens": len(token_ids), "completion_tokens": sum(len(r.output) for r in reqs)},
                "policy_version": engine.policy_version}

    @app.post("/inference/v1/prefill")
    async def prefill(body: dict):
        """Prefill role of a disaggregated deployment: runs the prompt and samples the first token. The K / V of the
        prompt are written to a file under ``kv_transfer_dir`` (shared memory on one box) and described in
        ``kv_transfer_params``, which the router passes on to a decode engine together with ``prefill_output``."""
        import os
        import tempfile
        import uuid

        token_ids = body.get("token_ids")
        if not token_ids:
            raise HTTPException(400, "token_ids is required")
        sp = dict(body.get("sampling_params") or {})
        sp.pop("n", None)
        params = SamplingParams.from_dict(sp)
        try:
            r = await engine.prefill(token_ids, params, str(body.get("cache_salt", "")))
        except NotImplementedError as e:
            raise HTTPException(501, str(e))
        kvp = None
        if r.finish_reason == "prefill_done" and r.handoff is not None:
            root = body.get("kv_transfer_dir") or ("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir())
            kvp = r.handoff.to_file(os.path.join(root, f"prb_kv_{uuid.uuid4().hex}.bin"))
            r.handoff = None
        return {"id": r.request_id, "model": body.get("model", model_name), "finish_reason": r.finish_reason,
                "prefill_output": {"token_ids": r.output, "logprobs": r.logprobs}, "kv_transfer_params": kvp,
                "usage": {"prompt_tokens": len(token_ids), "completion_tokens": len(r.output)},
                "policy_version": engine.policy_version}

    def _need_tokenizer():
        if tokenizer is None:
            raise HTTPException(501, "this server was started without a tokenizer; use /inference/v1/generate")

    @app.post("/v1/completions")
    async def completions(body: dict):
        _need_tokenizer()
        ids = tokenizer.encode(body["prompt"])
        params = SamplingParams.from_dict({"max_tokens": body.get("max_tokens", 16),
                                           "temperature": body.get("temperature", 1.0),
                                           "top_p": body.get("top_p", 1.0)})
        r = await engine.generate(ids, params, str(body.get("cache_salt", "")))
        return {"id": r.request_id, "object": "text_completion", "model": model_name,
                "choices": [{"index": 0, "text": tokenizer.decode(r.output), "finish_reason": r.finish_reason}]}

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        _need_tokenizer()
        ids = tokenizer.apply_chat_template(body["messages"], add_generation_prompt=True, tokenize=True)
        params = SamplingParams.from_dict({"max_tokens": body.get("max_tokens", body.get("max_completion_tokens", 256)),
                                           "temperature": body.get("temperature", 1.0),
                                           "top_p": body.get("top_p", 1.0)})
        r = await engine.generate(list(ids), params, str(body.get("cache_salt", "")))
        return {"id": r.request_id, "object": "chat.completion", "model": model_name,
                "choices": [{"index": 0, "finish_reason": r.finish_reason,
                             "message": {"role": "assistant", "content": tokenizer.decode(r.output)}}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(r.output)}}

    @app.post("/pause")
    async def pause():
        await asyncio.to_thread(engine.pause)
        return {"status": "paused"}

    @app.post("/resume")
    async def resume():
        engine.resume()
        return {"status": "running"}

    @app.post("/update_weights")
    async def update_weights(body: dict | None = None):
        weight_dir = (body or {}).get("weight_dir")
        was_paused = engine.paused
        if not was_paused:
            await asyncio.to_thread(engine.pause)
        try:
            if weight_dir is not None:
                await asyncio.to_thread(engine.update_weights_from_dir, weight_dir)
            elif engine.weight_receiver is not None:
                await asyncio.to_thread(engine.receive_weights)
            else:
                raise HTTPException(400, "weight_dir is null and no in-memory broadcaster was initialised")
        finally:
            if not was_paused:
                engine.resume()
        return {"status": "ok", "policy_version": engine.policy_version}

    @app.post("/init_broadcaster")
    async def init_broadcaster(body: dict):
        # NCCL: the engine's GPUs join the trainer's broadcast group; p2p: they publish where their parameter
        # storage can be written over NVLink peer memory. A tensor-parallel engine joins with every rank.
        await asyncio.to_thread(engine.init_broadcaster, body)
        return {"status": "ok"}

    @app.post("/load_lora_adapter")
    async def load_lora(body: dict):
        from ..models.lora_io import load_peft_adapter

        path = Path(body["lora_path"])
        was_paused = engine.paused
        if not was_paused:
            await asyncio.to_thread(engine.pause)
        try:
            await asyncio.to_thread(load_peft_adapter, engine.model, path)
            engine.cache.blocks.clear_prefix_cache()
            engine.policy_version += 1
        finally:
            if not was_paused:
                engine.resume()
        return {"status": "ok", "lora_name": body.get("lora_name")}

    return app
