"""Request router in front of several engine replicas (data-parallel rollout: one engine process
per GPU, every replica holds the whole model).

Generation requests go to ONE replica: requests that carry a ``cache_salt`` (or an ``x-session-id``
header) are placed by consistent hashing, so that the turns of one conversation meet their cached
prefix again; everything else goes to the replica with the fewest requests in flight. Admin
requests (pause / resume / weight updates / broadcaster setup / adapter loads) fan out to ALL
replicas and succeed only if every replica does; ``/health`` is healthy when all are; ``/metrics``
sums the replicas' counters and gauges.

Same role as the ``vllm-router`` subprocess the reference starts in front of its inference
replicas (src/prime_rl/entrypoints/inference.py:165-189) together with the client-side admin
fan-out (orchestrator/clients.py).
"""

import asyncio
import bisect
import hashlib
import json
import re

GENERATE_ROUTES = ("/inference/v1/generate", "/v1/completions", "/v1/chat/completions")
ADMIN_ROUTES = ("/pause", "/resume", "/update_weights", "/init_broadcaster", "/load_lora_adapter")


class HashRing:
    """Consistent hashing with virtual nodes: removing a replica only moves its own keys."""

    def __init__(self, nodes: list[int], vnodes: int = 64):
        self._ring: list[tuple[int, int]] = sorted(
            (self._h(f"{n}#{v}"), n) for n in nodes for v in range(vnodes))
        self._keys = [h for h, _ in self._ring]

    @staticmethod
    def _h(s: str) -> int:
        return int.from_bytes(hashlib.blake2b(s.encode(), digest_size=8).digest(), "big")

    def node(self, key: str) -> int:
        i = bisect.bisect(self._keys, self._h(key)) % len(self._ring)
        return self._ring[i][1]


class Router:
    def __init__(self, urls: list[str], transports: list | None = None, timeout: float = 3600.0,
                 prefill_urls: list[str] | None = None, prefill_transports: list | None = None):
        """``prefill_urls``: replicas that only run prompts (prefill / decode disaggregation). A generate request
        then goes to one of them first (``/inference/v1/prefill``); the K / V description and the first token it
        returns travel with the request to one of the decode replicas (``urls``), which continues from there."""
        import httpx

        if not urls:
            raise ValueError("the router needs at least one replica")
        self.urls = [u.rstrip("/") for u in urls]
        self.clients = [httpx.AsyncClient(base_url=u, timeout=timeout,
                                          transport=(transports[i] if transports else None))
                        for i, u in enumerate(self.urls)]
        self.prefill_urls = [u.rstrip("/") for u in (prefill_urls or [])]
        self.prefill_clients = [httpx.AsyncClient(base_url=u, timeout=timeout,
                                                  transport=(prefill_transports[i] if prefill_transports else None))
                                for i, u in enumerate(self.prefill_urls)]
        self.prefill_inflight = [0] * len(self.prefill_urls)
        self.handoffs = 0
        self.inflight = [0] * len(urls)
        self.served = [0] * len(urls)
        self.ring = HashRing(list(range(len(urls))))

    def pick(self, body: dict, headers) -> int:
        key = body.get("cache_salt") or headers.get("x-session-id")
        if key:
            return self.ring.node(str(key))
        return min(range(len(self.urls)), key=lambda i: (self.inflight[i], self.served[i]))

    async def _disaggregated(self, body: dict, headers) -> tuple[int, dict | str]:
        """One sample per hand-off: prefill replica (least loaded) -> decode replica (the usual choice)."""
        sp = dict(body.get("sampling_params") or {})
        n = int(sp.pop("n", 1) or 1)

        async def one():
            j = min(range(len(self.prefill_clients)), key=lambda i: self.prefill_inflight[i])
            self.prefill_inflight[j] += 1
            try:
                r = await self.prefill_clients[j].post("/inference/v1/prefill", json=dict(body, sampling_params=sp))
            finally:
                self.prefill_inflight[j] -= 1
            first = _payload(r)
            if r.status_code != 200:
                return r.status_code, first
            if not first.get("kv_transfer_params"):        # ended at its first token: nothing left to decode
                out = first["prefill_output"]
                return 200, {"id": first["id"], "model": first["model"], "policy_version": first.get("policy_version"),
                             "usage": first["usage"],
                             "choices": [{"index": 0, "token_ids": out["token_ids"], "logprobs": out["logprobs"],
                                          "finish_reason": first["finish_reason"], "prompt_logprobs": None,
                                          "routed_experts": None, "sampling_mask": None}]}
            self.handoffs += 1
            return await self._forward_to_decode("/inference/v1/generate",
                                                 dict(body, sampling_params=sp, prefill_output=first["prefill_output"],
                                                      kv_transfer_params=first["kv_transfer_params"]), headers)

        results = await asyncio.gather(*[one() for _ in range(n)])
        bad = next((r for r in results if r[0] != 200), None)
        if bad is not None:
            return bad
        merged = dict(results[0][1])
        merged["choices"] = [dict(r[1]["choices"][0], index=i) for i, r in enumerate(results)]
        merged["usage"] = {"prompt_tokens": results[0][1]["usage"]["prompt_tokens"],
                           "completion_tokens": sum(r[1]["usage"]["completion_tokens"] for r in results)}
        return 200, merged

    async def forward(self, path: str, body: dict, headers) -> tuple[int, dict | str]:
        if self.prefill_clients and path == "/inference/v1/generate" and not body.get("kv_transfer_params"):
            return await self._disaggregated(body, headers)
        return await self._forward_to_decode(path, body, headers)

    async def _forward_to_decode(self, path: str, body: dict, headers) -> tuple[int, dict | str]:
        i = self.pick(body, headers)
        self.inflight[i] += 1
        try:
            r = await self.clients[i].post(path, json=body)
        finally:
            self.inflight[i] -= 1
            self.served[i] += 1
        return r.status_code, _payload(r)

    async def fan_out(self, method: str, path: str, body: dict | None = None) -> list[tuple[int, dict | str]]:
        """Every replica gets the request; POST bodies that carry a ``rank_offset`` (weight-transfer
        group setup) get it advanced by the replica's index, so that replicas join as different ranks."""
        async def one(i, c):
            if method != "POST":
                r = await c.get(path)
            else:
                b = dict(body or {})
                if "rank_offset" in b or path == "/init_broadcaster":
                    b["rank_offset"] = int(b.get("rank_offset", 0)) + i
                r = await c.post(path, json=b)
            return r.status_code, _payload(r)

        # prefill replicas hold weights too: admin commands (pause, weight updates, ...) reach every engine
        return list(await asyncio.gather(*[one(i, c) for i, c in enumerate(self.clients + self.prefill_clients)]))

    async def close(self) -> None:
        await asyncio.gather(*[c.aclose() for c in self.clients + self.prefill_clients])


def _payload(r):
    try:
        return r.json()
    except Exception:
        return r.text


_METRIC = re.compile(r"^([a-zA-Z_:][\w:]*)(\{[^}]*\})?\s+([-+0-9.eE]+|NaN|[-+]?Inf)\s*$")


def merge_metrics(texts: list[str]) -> str:
    """Prometheus text of all replicas summed per (name, labels); comment lines kept once."""
    total: dict[str, float] = {}
    comments: list[str] = []
    for t in texts:
        for line in t.splitlines():
            if line.startswith("#"):
                if line not in comments:
                    comments.append(line)
                continue
            m = _METRIC.match(line.strip())
            if m:
                key = m.group(1) + (m.group(2) or "")
                try:
                    total[key] = total.get(key, 0.0) + float(m.group(3))
                except ValueError:
                    pass
    return "\n".join(comments + [f"{k} {v}" for k, v in total.items()]) + "\n"


def build_app(router: Router):
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, PlainTextResponse

    app = FastAPI(title="prime-rl-b200 inference router")
    app.state.router = router

    def reply(status: int, payload):
        if isinstance(payload, (dict, list)):
            return JSONResponse(payload, status_code=status)
        return PlainTextResponse(str(payload), status_code=status)

    for route in GENERATE_ROUTES:
        def make(route=route):
            async def handler(request: Request):
                body = await request.json()
                status, payload = await router.forward(route, body, request.headers)
                return reply(status, payload)
            return handler
        app.post(route)(make())

    for route in ADMIN_ROUTES:
        def make_admin(route=route):
            async def handler(request: Request):
                raw = await request.body()
                body = json.loads(raw) if raw else {}
                results = await router.fan_out("POST", route, body)
                bad = [(i, s, p) for i, (s, p) in enumerate(results) if s >= 400]
                if bad:
                    raise HTTPException(502, f"{route} failed on replicas {[i for i, _, _ in bad]}: {bad[0][2]}")
                return {"status": "ok", "replicas": len(results), "results": [p for _, p in results]}
            return handler
        app.post(route)(make_admin())

    @app.get("/health")
    async def health():
        results = await router.fan_out("GET", "/health")
        if any(s >= 400 for s, _ in results):
            raise HTTPException(503, "a replica is not healthy")
        return {"status": "ok", "replicas": len(results)}

    @app.get("/liveness")
    async def liveness():
        results = await router.fan_out("GET", "/liveness")
        if any(s >= 400 for s, _ in results):
            raise HTTPException(503, "a replica is not live")
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        r = await router.clients[0].get("/v1/models")
        return reply(r.status_code, _payload(r))

    @app.get("/metrics")
    async def metrics():
        results = await router.fan_out("GET", "/metrics")
        return PlainTextResponse(merge_metrics([p if isinstance(p, str) else json.dumps(p) for _, p in results]))

    @app.get("/router/state")
    async def state():
        return {"replicas": router.urls, "inflight": router.inflight, "served": router.served,
                "prefill_urls": router.prefill_urls, "prefill_inflight": router.prefill_inflight,
                "handoffs": router.handoffs}

    return app


def main(argv: list[str] | None = None) -> None:
    """``python -m prime_rl_b200.engine.router --port 8000 --backends http://a:9000,http://b:9000``: the router as a
    process of its own (multi-node serving: one router in front of the per-node servers)."""
    import argparse

    import uvicorn

    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--backends", required=True, help="comma-separated base URLs of the engine servers")
    ap.add_argument("--prefill-backends", default="", help="comma-separated base URLs of prefill-only engine servers "
                    "(prefill / decode disaggregation: --backends are then the decode engines)")
    ap.add_argument("--timeout", type=float, default=3600.0)
    args = ap.parse_args(argv)
    urls = [u for u in (x.strip() for x in args.backends.split(",")) if u]
    pre = [u for u in (x.strip() for x in args.prefill_backends.split(",")) if u]
    uvicorn.run(build_app(Router(urls, timeout=args.timeout, prefill_urls=pre)), host=args.host, port=args.port,
                log_level="warning")


if __name__ == "__main__":
    main()
