"""HTTP clients of the inference pool: token-in/token-out generation plus the admin plane
(health, pause / resume, weight updates, metrics), with per-attempt timeouts and retries
(reference: src/prime_rl/orchestrator/clients.py:77-504)."""

from __future__ import annotations

import asyncio
import base64
import os
import time

import httpx
import numpy as np


def _decode_routed(obj):
    if not obj:
        return None
    arr = np.frombuffer(base64.b64decode(obj["data"]), dtype=np.dtype(obj["dtype"])).reshape(obj["shape"])
    return arr


def _decode_mask(obj):
    if not obj:
        return None
    return (np.frombuffer(base64.b64decode(obj["ids"]), np.int32), np.frombuffer(base64.b64decode(obj["counts"]), np.int32))


class InferenceClient:
    def __init__(self, config, model_name: str, *, max_connections: int = 4096, retries: int = 3,
                 return_routed_experts: bool = False, return_sampling_mask: bool = False, transport=None):
        self.base = config.base_url.rstrip("/")
        self.root = self.base[:-3] if self.base.endswith("/v1") else self.base
        self.model_name, self.retries = model_name, retries
        headers = dict(config.headers)
        for h, var in config.headers_from_env.items():
            if os.getenv(var):
                headers[h] = os.environ[var]
        key = os.getenv(config.api_key_var)
        if key:
            headers["Authorization"] = f"Bearer {key}"
        limits = httpx.Limits(max_connections=max_connections, max_keepalive_connections=max_connections)
        self.http = httpx.AsyncClient(headers=headers, limits=limits, timeout=httpx.Timeout(600.0, connect=10.0),
                                      transport=transport)
        self.return_routed_experts, self.return_sampling_mask = return_routed_experts, return_sampling_mask

    async def _post(self, url: str, payload: dict, timeout: float | None = None) -> dict:
        last: Exception | None = None
        for attempt in range(self.retries):
            try:
                r = await self.http.post(url, json=payload, timeout=timeout)
                if r.status_code >= 500:
                    raise httpx.HTTPStatusError(f"{r.status_code}", request=r.request, response=r)
                r.raise_for_status()
                return r.json()
            except (httpx.TransportError, httpx.HTTPStatusError) as e:
                last = e
                if isinstance(e, httpx.HTTPStatusError) and e.response is not None and e.response.status_code < 500:
                    raise
                await asyncio.sleep(min(2.0 ** attempt * 0.2, 5.0))
        raise last  # type: ignore[misc]

    async def generate(self, token_ids: list[int], sampling, cache_salt: str = "", max_tokens: int | None = None,
                       mm: dict | None = None) -> dict:
        sp = {"temperature": sampling.temperature, "top_p": sampling.top_p,
              "max_tokens": max_tokens or sampling.max_completion_tokens or 128, "logprobs": 0}
        if getattr(sampling, "top_k", None):
            sp["top_k"] = sampling.top_k
        sp.update(getattr(sampling, "extra_body", {}) or {})
        if self.return_routed_experts:
            sp["return_routed_experts"] = True
        body = {"model": self.model_name, "token_ids": token_ids, "sampling_params": sp, "cache_salt": cache_salt,
                "return_sampling_mask": self.return_sampling_mask}
        if mm is not None:
            import base64

            import numpy as np

            px = np.ascontiguousarray(np.asarray(mm["pixel_values"], dtype=np.float32))
            body["multi_modal_data"] = {"pixel_values": {"dtype": "float32", "shape": list(px.shape),
                                                         "data": base64.b64encode(px.tobytes()).decode()},
                                        "image_grid_thw": [list(map(int, g)) for g in mm["image_grid_thw"]]}
        out = await self._post(f"{self.root}/inference/v1/generate", body)
        ch = out["choices"][0]
        return {"token_ids": ch["token_ids"], "logprobs": ch["logprobs"], "finish_reason": ch.get("finish_reason"),
                "routed_experts": _decode_routed(ch.get("routed_experts")),
                "sampling_mask": _decode_mask(ch.get("sampling_mask")),
                "policy_version": out.get("policy_version")}

    async def prompt_logprobs(self, token_ids: list[int]) -> list[float]:
        body = {"model": self.model_name, "token_ids": token_ids,
                "sampling_params": {"max_tokens": 1, "temperature": 0.0, "prompt_logprobs": True}}
        out = await self._post(f"{self.root}/inference/v1/generate", body)
        return out["choices"][0]["prompt_logprobs"]

    async def close(self) -> None:
        await self.http.aclose()


class AdminPlane:
    """Admin operations against every engine replica directly (bypassing routers)."""

    def __init__(self, config, transport=None):
        urls = config.admin_base_url or [config.base_url]
        self.roots = [u.rstrip("/")[:-3] if u.rstrip("/").endswith("/v1") else u.rstrip("/") for u in urls]
        self.http = httpx.AsyncClient(timeout=httpx.Timeout(1800.0, connect=10.0), transport=transport)
        self.ready_timeout = config.wait_for_ready_timeout

    async def _all(self, method: str, path: str, **kw):
        async def one(root):
            r = await self.http.request(method, root + path, **kw)
            r.raise_for_status()
            return r
        return await asyncio.gather(*[one(r) for r in self.roots])

    async def wait_for_ready(self) -> None:
        t0 = time.monotonic()
        while True:
            try:
                await self._all("GET", "/health", timeout=5.0)
                return
            except Exception:
                if time.monotonic() - t0 > self.ready_timeout:
                    raise TimeoutError(f"inference pool not ready after {self.ready_timeout}s")
                await asyncio.sleep(0.5)

    async def pause(self):
        await self._all("POST", "/pause")

    async def resume(self):
        await self._all("POST", "/resume")

    async def update_weights(self, weight_dir: str | None):
        await self._all("POST", "/update_weights", json={"weight_dir": weight_dir})

    async def load_lora_adapter(self, name: str, path: str):
        await self._all("POST", "/load_lora_adapter", json={"lora_name": name, "lora_path": path})

    async def init_broadcaster(self, **kw):
        async def one(i, root):
            body = dict(kw, rank_offset=i)
            r = await self.http.post(root + "/init_broadcaster", json=body)
            r.raise_for_status()
        await asyncio.gather(*[one(i, r) for i, r in enumerate(self.roots)])

    async def metrics(self) -> list[dict[str, float]]:
        out = []
        for r in await self._all("GET", "/metrics", timeout=5.0):
            d = {}
            for line in r.text.splitlines():
                if line and not line.startswith("#"):
                    k, _, v = line.rpartition(" ")
                    try:
                        d[k.split("{")[0]] = float(v)
                    except ValueError:
                        pass
            out.append(d)
        return out

    async def close(self):
        await self.http.aclose()
