"""Environment server and its client: an ``Environment`` served over HTTP so that task
generation and scoring can run on other machines than the orchestrator (the reference's
``env-server`` serves a verifiers environment the same way; src/prime_rl/entrypoints/env_server.py).

    GET  /info                       -> {"name", "num_tasks"}
    POST /task   {"task_id": n}      -> the task dict (token-level prompt and scoring payload)
    POST /score  {"task", "completion"} -> {"reward": float}
"""

from __future__ import annotations

import asyncio
from typing import Any

import httpx

from .envs import Environment, load_environment


def build_app(env: Environment):
    from fastapi import FastAPI

    app = FastAPI(title=f"env-server:{env.name}")

    @app.get("/info")
    def info():
        return {"name": env.name, "num_tasks": env.num_tasks}

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.post("/task")
    def task(body: dict):
        return env.task(int(body["task_id"]))

    @app.post("/score")
    def score(body: dict):
        return {"reward": float(env.score(body["task"], list(body["completion"])))}

    return app


def serve(config) -> None:
    import uvicorn

    env = load_environment(config.env)
    uvicorn.run(build_app(env), host=config.serve.host, port=config.serve.port, log_level=(config.log.level or "info"),
                limit_concurrency=config.serve.max_concurrent)


class RemoteEnvironment(Environment):
    """Client side: tasks and scores come from an env server; rollouts run here against the
    inference client like any local environment."""

    def __init__(self, base_url: str, name: str | None = None, transport=None, **kw):
        self.base = base_url.rstrip("/")
        self._http = httpx.Client(timeout=60.0, transport=transport)
        info = self._http.get(f"{self.base}/info").json()
        super().__init__(name=name or info["name"], num_tasks=info["num_tasks"], **kw)

    def task(self, task_id: int) -> dict[str, Any]:
        return self._http.post(f"{self.base}/task", json={"task_id": task_id}).json()

    def score(self, task: dict[str, Any], completion: list[int]) -> float:
        return float(self._http.post(f"{self.base}/score", json={"task": task, "completion": completion}).json()["reward"])

    async def rollout(self, client, task_id, sampling, policy_version, group_id):
        # task fetch and scoring are blocking HTTP calls: keep them off the event loop
        loop = asyncio.get_running_loop()
        task = await loop.run_in_executor(None, self.task, task_id)
        from .types import Rollout, Turn

        out = await client.generate(task["prompt"], sampling, cache_salt=str(policy_version))
        turn = Turn(task["prompt"], out["token_ids"], out["logprobs"], temperature=sampling.temperature,
                    routed_experts=out.get("routed_experts"), sampling_mask=out.get("sampling_mask"),
                    finish_reason=out.get("finish_reason"))
        reward = await loop.run_in_executor(None, self.score, task, out["token_ids"])
        return Rollout(env_name=self.name, task_id=task_id, group_id=group_id, turns=[turn], reward=reward,
                       policy_version=out.get("policy_version", policy_version), metrics={"reward": reward})
