"""``dashboard [dir ...] [--port N]``: serves the run dashboard for the given output
directories plus everything launchers have registered
(reference: src/prime_rl/entrypoints/dashboard.py)."""

from __future__ import annotations

import argparse
from pathlib import Path


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("dirs", nargs="*", type=Path)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8765)
    args = ap.parse_args(argv)
    import uvicorn

    from ..dashboard.server import build_app, register_output_dir

    for d in args.dirs:
        register_output_dir(d)
    uvicorn.run(build_app([str(d.resolve()) for d in args.dirs]), host=args.host, port=args.port, log_level="warning")


if __name__ == "__main__":
    main()
