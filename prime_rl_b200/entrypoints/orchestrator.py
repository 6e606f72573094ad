"""``orchestrator @ orchestrator.toml``: the asynchronous rollout orchestrator process."""

from ..orchestrator.orchestrator import main

if __name__ == "__main__":
    main()
