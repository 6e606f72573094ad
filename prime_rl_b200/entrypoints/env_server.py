"""``env-server @ env.toml``: serves one environment over HTTP
(reference: src/prime_rl/entrypoints/env_server.py)."""

from __future__ import annotations

from ..configs.base import cli
from ..configs.evals import EnvServerConfig


def main(argv: list[str] | None = None) -> None:
    config = cli(EnvServerConfig, argv)
    from ..orchestrator.env_server import serve

    serve(config)


if __name__ == "__main__":
    main()
