"""``sft @ sft.toml``: launches the SFT trainer under ``torch.distributed.run`` on the local
GPUs, or renders and submits a SLURM script when ``slurm`` / a multi-node deployment is
configured (reference: src/prime_rl/entrypoints/sft.py).

The resolved config is written to ``<output_dir>/configs/attempt_N/resolved/sft.json`` first;
``--dry-run`` stops there.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

from ..configs.base import cli
from ..configs.sft import SFTConfig
from ..utils.logger import setup_logger
from ..utils.pathing import prepare_attempt_dirs


def _num_gpus(config: SFTConfig) -> int:
    dep = config.deployment
    n = getattr(dep, "num_gpus", None) or getattr(dep, "num_train_gpus", None)
    if n:
        return int(n)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        return len([x for x in visible.split(",") if x])
    try:
        import torch

        return max(1, torch.cuda.device_count())
    except Exception:
        return 1


def main(argv: list[str] | None = None) -> None:
    config = cli(SFTConfig, argv)
    log = setup_logger(config.log.level or "info", tag="sft")
    out = config.output_dir
    if config.clean and out.exists():
        shutil.rmtree(out)
    out.mkdir(parents=True, exist_ok=True)
    attempt, cfg_dir, log_dir = prepare_attempt_dirs(out)
    cfg_path = cfg_dir / "sft.json"
    config.dump(cfg_path)
    multi_node = getattr(config.deployment, "type", "single_node") == "multi_node"
    if config.slurm is not None or multi_node:
        from ..utils.slurm import render_sft_sbatch

        nodes = getattr(config.deployment, "num_nodes", None) or getattr(config.deployment, "num_train_nodes", 1)
        gpn = getattr(config.deployment, "gpus_per_node", 8)
        if config.slurm is None:
            from ..configs.shared import SlurmConfig

            config.slurm = SlurmConfig()
        script = out / "sft.sbatch"
        script.write_text(render_sft_sbatch(_RunDirView(config, out), cfg_path, nodes=nodes, gpus_per_node=gpn))
        log.info(f"wrote {script}")
        if config.dry_run:
            return
        sys.exit(subprocess.call(["sbatch", str(script)]))
    log.info(f"output dir {out} (attempt {attempt})")
    if config.dry_run:
        log.info("dry run: resolved config written, not launching")
        return
    n = _num_gpus(config)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29500 + attempt % 100), "-m", "prime_rl_b200.trainer.sft.train", "@",
           str(cfg_path)]
    env = dict(os.environ, PYTHONUNBUFFERED="1", PRL_LOG_DIR=str(log_dir))
    with open(log_dir / "sft.log", "w") as f:
        rc = subprocess.call(cmd, env=env, stdout=f, stderr=subprocess.STDOUT)
    if rc != 0:
        log.error(f"sft trainer exited with code {rc}; see {log_dir}/sft.log")
    sys.exit(rc)


class _RunDirView:
    """What the sbatch renderer reads from a config: ``slurm``, ``run_dir``, ``env_vars``."""

    def __init__(self, config: SFTConfig, run_dir):
        self.slurm, self.run_dir = config.slurm, run_dir
        self.env_vars = getattr(config, "env_vars", {})


if __name__ == "__main__":
    main()
