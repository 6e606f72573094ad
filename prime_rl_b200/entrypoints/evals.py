"""``evals @ evals.toml``: standalone online evaluation against a running inference server
(reference: src/prime_rl/entrypoints/evals.py). The resolved config goes to
``<output_dir>/configs/attempt_N/resolved/evals.json``."""

from __future__ import annotations

import asyncio

from ..configs.base import cli
from ..configs.evals import EvalsConfig
from ..utils.pathing import prepare_attempt_dirs


def main(argv: list[str] | None = None) -> None:
    config = cli(EvalsConfig, argv)
    config.output_dir.mkdir(parents=True, exist_ok=True)
    _, cfg_dir, _ = prepare_attempt_dirs(config.output_dir)
    config.dump(cfg_dir / "evals.json")
    if config.dry_run:
        return
    from ..evals.evals import run_evals

    asyncio.run(run_evals(config))


if __name__ == "__main__":
    main()
