"""sbatch script rendering for the ``rl`` / ``sft`` / ``inference`` launchers.

The reference ships Jinja templates (src/prime_rl/templates/{single_node_rl,multi_node_rl,
single_node_sft,multi_node_sft,inference}.sbatch.j2); the scripts here have the same structure
(one job, ``srun`` per role, trainer under ``torch.distributed.run`` with the first train node as
rendezvous host, inference replicas on their own nodes, orchestrator on the first train node or
the first inference node) but are plain Python string assembly, so the launcher has no template
dependency. A user template (``slurm.template_path``) is filled with ``str.format_map``.
"""

from __future__ import annotations

import shlex
from pathlib import Path


def _header(slurm, nodes: int, gpus_per_node: int, log_dir: Path) -> list[str]:
    lines = ["#!/bin/bash", f"#SBATCH --job-name={slurm.job_name}", f"#SBATCH --nodes={nodes}",
             f"#SBATCH --gres=gpu:{gpus_per_node}", "#SBATCH --ntasks-per-node=1", "#SBATCH --exclusive",
             f"#SBATCH --partition={slurm.partition}", f"#SBATCH --output={log_dir}/slurm-%j.out",
             f"#SBATCH --error={log_dir}/slurm-%j.err"]
    for key in ("nodelist", "exclude", "account", "time"):
        val = getattr(slurm, key, None)
        if val:
            lines.append(f"#SBATCH --{key}={val}")
    lines += ["", "set -euo pipefail", f"cd {shlex.quote(str(Path(slurm.project_dir).resolve()))}",
              'NODES=($(scontrol show hostnames "$SLURM_JOB_NODELIST"))', 'HEAD=${NODES[0]}',
              'export MASTER_ADDR=$HEAD', 'export MASTER_PORT=${MASTER_PORT:-29400}', 'export PYTHONUNBUFFERED=1']
    if slurm.pre_run_command:
        lines.append(slurm.pre_run_command)
    return lines


def _cleanup(grace: int) -> list[str]:
    return ["", "cleanup() {", "  trap - TERM INT EXIT", "  kill $(jobs -p) 2>/dev/null || true",
            f"  sleep {min(grace, 30)}", "}", "trap cleanup TERM INT EXIT"]


def _env_exports(env_vars: dict) -> list[str]:
    return [f"export {k}={shlex.quote(str(v))}" for k, v in (env_vars or {}).items()]


def render_rl_sbatch(config, paths: dict) -> str:
    """``paths``: sub-config files written by the launcher (keys trainer / orchestrator / inference)."""
    slurm = config.slurm
    dep = config.deployment
    log_dir = Path(config.run_dir) / "logs"
    if getattr(dep, "type", "single_node") == "multi_node":
        gpn = dep.gpus_per_node
        n_train = dep.num_train_nodes
        n_infer = dep.num_infer_nodes if dep.num_infer_nodes is not None else 0
        nodes = n_train + n_infer
    else:
        gpn, n_train, n_infer, nodes = 8, 1, 0, 1
    if slurm is None:
        from ..configs.shared import SlurmConfig

        slurm = SlurmConfig()
    if slurm.template_path:
        return Path(slurm.template_path).read_text().format_map(
            dict(slurm.template_vars, nodes=nodes, gpus_per_node=gpn, num_train_nodes=n_train,
                 num_infer_nodes=n_infer, trainer_config=paths["trainer"], orchestrator_config=paths["orchestrator"],
                 inference_config=paths.get("inference", ""), log_dir=log_dir))
    L = _header(slurm, nodes, gpn, log_dir) + _env_exports(config.env_vars) + _cleanup(slurm.cleanup_grace_period)
    L += ["", f"mkdir -p {log_dir}"]
    if nodes == 1:
        # everything on one node: the local launcher splits the GPUs itself
        L += ["", f"srun --nodes=1 --ntasks=1 python -m prime_rl_b200.entrypoints.rl @ {paths.get('rl', paths['trainer'])} "
                  f"--slurm None > {log_dir}/rl.log 2>&1"]
        return "\n".join(L) + "\n"
    L += ["", f"TRAIN_NODES=(\"${{NODES[@]:0:{n_train}}}\")", f"INFER_NODES=(\"${{NODES[@]:{n_train}:{n_infer}}}\")",
          'TRAIN_HEAD=${TRAIN_NODES[0]}', 'export MASTER_ADDR=$TRAIN_HEAD']
    if "inference" in paths and n_infer > 0:
        per = max(1, n_infer // max(1, dep.num_infer_replicas))
        L += ["", "# inference replicas", f"REPLICA_NODES={per}", "for ((r = 0; r < ${#INFER_NODES[@]}; r += REPLICA_NODES)); do",
              "  node=${INFER_NODES[$r]}",
              f"  srun --nodes=1 --ntasks=1 -w $node python -m prime_rl_b200.entrypoints.inference @ {paths['inference']} "
              f"> {log_dir}/inference_$node.log 2>&1 &", "done",
              'INFER_URLS=$(printf "http://%s:8000/v1," "${INFER_NODES[@]}")', 'export PRL_INFERENCE_URLS=${INFER_URLS%,}']
    orch_node = "${INFER_NODES[0]}" if (dep.orchestrator_on_inference and n_infer > 0) else "$TRAIN_HEAD"
    L += ["", "# orchestrator (CPU only)",
          f"srun --nodes=1 --ntasks=1 --overlap -w {orch_node} env CUDA_VISIBLE_DEVICES= python -m "
          f"prime_rl_b200.entrypoints.orchestrator @ {paths['orchestrator']} > {log_dir}/orchestrator.log 2>&1 &",
          "", "# trainer: one torch.distributed.run agent per train node",
          f"srun --nodes={n_train} --ntasks={n_train} -w $(IFS=,; echo \"${{TRAIN_NODES[*]}}\") bash -c '"
          f"python -m torch.distributed.run --nnodes={n_train} --nproc-per-node={gpn} --node-rank=$SLURM_NODEID "
          f"--master-addr=$MASTER_ADDR --master-port=$MASTER_PORT -m prime_rl_b200.trainer.rl.train @ {paths['trainer']}' "
          f"> {log_dir}/trainer.log 2>&1 &", "", "wait -n", "exit $?"]
    return "\n".join(L) + "\n"


def render_sft_sbatch(config, trainer_config: Path, nodes: int = 1, gpus_per_node: int = 8) -> str:
    slurm = config.slurm
    log_dir = Path(config.run_dir) / "logs"
    L = _header(slurm, nodes, gpus_per_node, log_dir) + _env_exports(getattr(config, "env_vars", {})) + \
        _cleanup(slurm.cleanup_grace_period)
    L += ["", f"mkdir -p {log_dir}",
          f"srun --nodes={nodes} --ntasks={nodes} bash -c 'python -m torch.distributed.run --nnodes={nodes} "
          f"--nproc-per-node={gpus_per_node} --node-rank=$SLURM_NODEID --master-addr=$MASTER_ADDR "
          f"--master-port=$MASTER_PORT -m prime_rl_b200.trainer.sft.train @ {trainer_config}' > {log_dir}/sft.log 2>&1"]
    return "\n".join(L) + "\n"


def render_inference_sbatch(config, inference_config: Path, nodes: int = 1, gpus_per_node: int = 8) -> str:
    slurm = config.slurm
    log_dir = Path(getattr(config, "run_dir", Path("outputs"))) / "logs"
    L = _header(slurm, nodes, gpus_per_node, log_dir) + _cleanup(slurm.cleanup_grace_period)
    L += ["", f"mkdir -p {log_dir}", "for node in \"${NODES[@]}\"; do",
          f"  srun --nodes=1 --ntasks=1 -w $node python -m prime_rl_b200.entrypoints.inference @ {inference_config} "
          f"> {log_dir}/inference_$node.log 2>&1 &", "done", "wait"]
    return "\n".join(L) + "\n"
