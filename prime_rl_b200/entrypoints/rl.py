"""``rl @ rl.toml``: launches inference, orchestrator and trainer as supervised child
processes on one node (GPU ids split between inference and trainer), or renders a SLURM
script for multi-node runs (reference: src/prime_rl/entrypoints/rl.py:116-698).

    configs/attempt_N/resolved/{rl,trainer,orchestrator,inference}.json are written first;
    ``--dry-run`` stops there.
"""

from __future__ import annotations

import os
import shutil
import sys
import uuid
from pathlib import Path

from ..configs.base import cli
from ..configs.rl import MultiNodeDeploymentConfig, RLConfig
from ..utils.logger import setup_logger
from ..utils.pathing import clean_future_steps, get_ckpt_dir, latest_step, prepare_attempt_dirs
from ..utils.process import Supervisor, popen


def write_subconfigs(config: RLConfig, cfg_dir: Path) -> dict[str, Path]:
    paths = {"rl": cfg_dir / "rl.json", "trainer": cfg_dir / "trainer.json",
             "orchestrator": cfg_dir / "orchestrator.json"}
    config.dump(paths["rl"])
    config.trainer.dump(paths["trainer"])
    config.orchestrator.dump(paths["orchestrator"])
    if config.inference is not None:
        paths["inference"] = cfg_dir / "inference.json"
        config.inference.dump(paths["inference"])
    return paths


def prepare_env_servers(config: RLConfig, cfg_dir: Path) -> list[tuple[str, Path, str]]:
    """One ``envs/<kind>-<name>.json`` (an ``EnvServerConfig``) per source that gets a server of its own; the
    orchestrator's source is re-pointed at the server's address. Returns (label, config file, address)."""
    from urllib.parse import urlparse

    out = []
    env_dir = cfg_dir / "envs"
    for kind, src, addr in config.orchestrator.spawned_sources():
        env_dir.mkdir(parents=True, exist_ok=True)
        u = urlparse(addr)
        spec = {"env": {"id": src.id, "import_path": src.import_path, "args": src.args, "name": src.resolved_name},
                "serve": {"host": u.hostname or "127.0.0.1", "port": u.port or 80},
                "log": {"level": config.log.level} if config.log.level else {}}
        path = env_dir / f"{kind}-{src.resolved_name}.json"
        import json

        path.write_text(json.dumps(spec, indent=2))
        src.name = src.resolved_name
        src.id, src.import_path, src.args = "remote", None, {"base_url": addr}
        out.append((f"env-{kind}-{src.name}", path, addr))
    return out


def wait_for_http(url: str, timeout: float = 120.0) -> None:
    import time
    import urllib.request

    t0 = time.monotonic()
    while True:
        try:
            with urllib.request.urlopen(url, timeout=2.0) as r:
                if r.status == 200:
                    return
        except OSError:
            pass
        if time.monotonic() - t0 > timeout:
            raise TimeoutError(f"{url} did not answer within {timeout}s")
        time.sleep(0.2)


def gpu_split(config: RLConfig) -> tuple[list[int], list[int]]:
    d = config.deployment
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    ids = [int(x) for x in visible.split(",")] if visible else list(range(d.num_infer_gpus + d.num_train_gpus))
    n_inf = d.num_infer_gpus if config.inference is not None else 0
    return ids[:n_inf], ids[n_inf:n_inf + d.num_train_gpus]


def rl_local(config: RLConfig) -> int:
    log = setup_logger(config.log.level or "info", tag="rl")
    run_dir = config.run_dir
    if config.clean and run_dir.exists():
        shutil.rmtree(run_dir)
    run_dir.mkdir(parents=True, exist_ok=True)
    attempt, cfg_dir, log_dir = prepare_attempt_dirs(run_dir)
    env_servers = prepare_env_servers(config, cfg_dir)          # before the orchestrator's config is written
    paths = write_subconfigs(config, cfg_dir)
    log.info(f"run dir {run_dir} (attempt {attempt})")
    if config.dry_run:
        log.info("dry run: resolved configs written, not launching")
        return 0
    if config.resume is not None:
        step = config.resume.step if config.resume.step is not None else latest_step(get_ckpt_dir(run_dir))
        clean_future_steps(run_dir, step)
    infer_gpus, train_gpus = gpu_split(config)
    base_env = dict(os.environ, PRL_RUN_ID=os.environ.get("PRL_RUN_ID", uuid.uuid4().hex),
                    PRL_RUN_NAME=config.run.name or "", PYTHONUNBUFFERED="1")
    base_env.update(config.env_vars)
    py = sys.executable
    sup = Supervisor()
    try:
        if config.inference is not None:
            env = dict(base_env, **config.inference.env_vars, CUDA_VISIBLE_DEVICES=",".join(map(str, infer_gpus)))
            sup.add("inference", popen([py, "-m", "prime_rl_b200.entrypoints.inference", "@", str(paths["inference"])],
                                       env, log_dir / "inference.log"))
        for label, path, addr in env_servers:
            env = dict(base_env, **config.orchestrator.env_vars, CUDA_VISIBLE_DEVICES="")
            sup.add(label, popen([py, "-m", "prime_rl_b200.entrypoints.env_server", "@", str(path)], env,
                                 log_dir / f"{label}.log"))
        for label, _, addr in env_servers:
            wait_for_http(addr.rstrip("/") + "/health")
        env = dict(base_env, **config.orchestrator.env_vars, CUDA_VISIBLE_DEVICES="")
        sup.add("orchestrator", popen([py, "-m", "prime_rl_b200.entrypoints.orchestrator", "@",
                                       str(paths["orchestrator"])], env, log_dir / "orchestrator.log"))
        n = max(1, len(train_gpus))
        env = dict(base_env, **config.trainer.env_vars, CUDA_VISIBLE_DEVICES=",".join(map(str, train_gpus)))
        cmd = [py, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
               "--master-port", str(29400 + attempt % 100), "-m", "prime_rl_b200.trainer.rl.train", "@",
               str(paths["trainer"])]
        sup.add("trainer", popen(cmd, env, log_dir / "trainer.log"))
        failure = sup.wait(required=["trainer", "orchestrator"])
        if failure is not None:
            log.error(f"{failure[0]} exited with code {failure[1]}; see {log_dir}/{failure[0]}.log")
            return failure[1] or 1
        log.info("trainer and orchestrator finished")
        return 0
    finally:
        sup.shutdown()


def rl_slurm(config: RLConfig) -> int:
    from ..utils.slurm import render_rl_sbatch

    run_dir = config.run_dir
    run_dir.mkdir(parents=True, exist_ok=True)
    _, cfg_dir, _ = prepare_attempt_dirs(run_dir)
    paths = write_subconfigs(config, cfg_dir)
    script = run_dir / "rl.sbatch"
    script.write_text(render_rl_sbatch(config, paths))
    print(f"wrote {script}")
    if config.dry_run:
        return 0
    import subprocess

    return subprocess.call(["sbatch", str(script)])


def main(argv: list[str] | None = None) -> None:
    config = cli(RLConfig, argv)
    if config.slurm is not None or isinstance(config.deployment, MultiNodeDeploymentConfig):
        sys.exit(rl_slurm(config))
    sys.exit(rl_local(config))


if __name__ == "__main__":
    main()
