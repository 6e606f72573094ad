"""sbatch script rendering for the ``rl`` / ``sft`` / ``inference`` launchers.

Scripts are Jinja templates under ``prime_rl_b200/templates`` (own text; same roles and the same template
variable names as the reference's src/prime_rl/templates/{single_node_rl,multi_node_rl,single_node_sft,
multi_node_sft,inference}.sbatch.j2, so a user template written for those variables, given as
``slurm.template_path``, renders here too). Structure of a multi-node RL job:

* one ``srun`` task per node, ``--kill-on-bad-exit=1``; the node's role follows from ``SLURM_PROCID``: the first
  ``num_infer_nodes`` tasks serve inference (every node its own data-parallel replicas, one router on the first
  node in front of all of them), the rest run one ``torch.distributed.run`` agent each;
* the orchestrator and the environment servers run beside trainer rank 0, or on the last inference node with
  ``deployment.orchestrator_on_inference``;
* the trainer and the orchestrator leave marker files when they end cleanly; every node stays up until all
  markers exist, so inference keeps serving while either still runs, and a component that fails ends the job
  after ``slurm.cleanup_grace_period`` seconds (time for a checkpoint in flight elsewhere);
* pids of everything a node starts are recorded under the run directory, and the next job ends exactly those
  leftovers before it starts (nothing is matched by process name).
"""

from __future__ import annotations

import shlex
from pathlib import Path

TEMPLATE_DIR = Path(__file__).resolve().parents[1] / "templates"


def _environment(extra_dir: Path | None = None):
    import jinja2

    search = [str(TEMPLATE_DIR)] + ([str(extra_dir)] if extra_dir else [])
    env = jinja2.Environment(loader=jinja2.FileSystemLoader(search), undefined=jinja2.StrictUndefined,
                             keep_trailing_newline=True, trim_blocks=False, lstrip_blocks=False)
    env.filters["shq"] = lambda v: shlex.quote(str(v))
    return env


def _render(name: str, slurm, variables: dict) -> str:
    """Renders the stock template ``name`` or, when ``slurm.template_path`` is set, the user's file (which may
    ``{% include %}`` the stock pieces)."""
    user = getattr(slurm, "template_path", None)
    if user:
        user = Path(user)
        env = _environment(user.parent)
        return env.from_string(user.read_text()).render(**variables)
    return _environment().get_template(name).render(**variables)


def _common(slurm, run_dir: Path, total_nodes: int, gpus_per_node: int, env_vars: dict | None,
            ranks_filter=(0,)) -> dict:
    if slurm is None:
        from ..configs.shared import SlurmConfig

        slurm = SlurmConfig()
    run_dir = Path(run_dir)
    launcher_dir = run_dir / "launcher"
    return {
        "job_name": slurm.job_name, "partition": slurm.partition, "project_dir": str(Path(slurm.project_dir).resolve()),
        "account": slurm.account, "time": slurm.time, "nodelist": slurm.nodelist, "exclude": slurm.exclude,
        "slurm_opts": {k: getattr(slurm, k, None) for k in ("account", "time", "nodelist", "exclude")},
        "pre_run_command": slurm.pre_run_command, "cleanup_grace_period": int(slurm.cleanup_grace_period),
        "shared_fs": slurm.shared_fs, "total_nodes": total_nodes, "gpus_per_node": gpus_per_node,
        "output_dir": str(run_dir), "log_dir": str(run_dir / "logs"), "launcher_dir": str(launcher_dir),
        "launcher_log_dir": str(launcher_dir / "logs"), "env_vars": dict(env_vars or {}),
        "ranks_filter": ",".join(str(r) for r in ranks_filter),
    }


def _inference_vars(inference, gpus_per_node: int) -> dict:
    """Placement of the inference servers: replicas per node, ports, prefill / decode split."""
    out = {"is_disaggregated": False, "num_prefill_nodes": 0, "num_decode_nodes": 0, "prefill_port": 8100,
           "decode_port": 8200, "prefill_env_vars": {}, "decode_env_vars": {}, "inference_tp": 1,
           "dp_per_node": gpus_per_node, "router_port": 8000, "backend_port": 8001, "nodes_per_infer_replica": 1,
           "inference_data_parallel_rpc_port": 13345}
    if inference is None:
        return out
    tp = max(1, inference.vllm.tensor_parallel_size)
    out.update(inference_tp=tp, dp_per_node=max(1, gpus_per_node // tp), router_port=inference.server.port,
               backend_port=inference.server.port + 1000,
               inference_data_parallel_rpc_port=inference.vllm.data_parallel_rpc_port)
    dep = getattr(inference, "deployment", None)
    kind = getattr(dep, "type", "single_node")
    if kind == "multi_node":
        out["nodes_per_infer_replica"] = dep.num_nodes
    elif kind == "disaggregated":
        out.update(is_disaggregated=True,
                   num_prefill_nodes=dep.prefill_nodes_per_replica * dep.num_prefill_replicas,
                   num_decode_nodes=dep.decode_nodes_per_replica * dep.num_decode_replicas,
                   prefill_port=dep.prefill_port, decode_port=dep.decode_port,
                   prefill_env_vars=dict(dep.prefill_env_vars), decode_env_vars=dict(dep.decode_env_vars),
                   nodes_per_infer_replica=dep.prefill_nodes_per_replica + dep.decode_nodes_per_replica)
    return out


def render_rl_sbatch(config, paths: dict) -> str:
    """``paths``: sub-config files written by the launcher (keys rl / trainer / orchestrator / inference); the
    templates address them through their common directory."""
    dep = config.deployment
    multi = getattr(dep, "type", "single_node") == "multi_node"
    gpn = dep.gpus_per_node
    n_train = dep.num_train_nodes if multi else 1
    n_infer = (dep.num_infer_nodes or 0) if multi else 0
    if config.inference is None:
        n_infer = 0
    config_dir = Path(paths["trainer"]).parent
    v = _common(config.slurm, config.run_dir, n_train + n_infer if multi else 1, gpn, config.env_vars,
                getattr(config.trainer.log, "ranks_filter", [0]))
    v.update(_inference_vars(config.inference, gpn))
    wb, rt_ = config.trainer.weight_broadcast, getattr(config.trainer, "rollout_transport", None)
    sources = list(config.orchestrator.spawned_sources()) if hasattr(config.orchestrator, "spawned_sources") else []
    v.update(
        config_dir=str(config_dir), config_path=str(paths.get("rl", paths["trainer"])),
        num_train_nodes=n_train, num_infer_nodes=n_infer,
        num_infer_replicas=getattr(dep, "num_infer_replicas", 1),
        orchestrator_on_inference=bool(getattr(dep, "orchestrator_on_inference", False)),
        trainer_env_vars=dict(config.trainer.env_vars), orchestrator_env_vars=dict(config.orchestrator.env_vars),
        inference_env_vars=dict(config.inference.env_vars) if config.inference is not None else {},
        use_nccl_broadcast=getattr(wb, "type", None) == "nccl", use_nixl_broadcast=getattr(wb, "type", None) == "nixl",
        use_zmq_transport=getattr(rt_, "type", None) == "zmq",
        train_env_names=[f"{kind}-{src.resolved_name}" for kind, src, _ in sources if kind == "train"],
        eval_env_names=[f"{kind}-{src.resolved_name}" for kind, src, _ in sources if kind != "train"],
    )
    return _render("multi_node_rl.sbatch.j2" if multi else "single_node_rl.sbatch.j2", config.slurm, v)


def render_sft_sbatch(config, trainer_config: Path, nodes: int = 1, gpus_per_node: int = 8) -> str:
    v = _common(config.slurm, config.run_dir, nodes, gpus_per_node, getattr(config, "env_vars", {}),
                getattr(getattr(config, "log", None), "ranks_filter", [0]))
    v.update(config_path=str(trainer_config), config_dir=str(Path(trainer_config).parent), num_nodes=nodes)
    return _render("multi_node_sft.sbatch.j2" if nodes > 1 else "single_node_sft.sbatch.j2", config.slurm, v)


def render_inference_sbatch(config, inference_config: Path, nodes: int = 1, gpus_per_node: int = 8) -> str:
    run_dir = getattr(config, "run_dir", None) or getattr(config, "output_dir", None) or Path("outputs")
    v = _common(config.slurm, run_dir, nodes, gpus_per_node, getattr(config, "env_vars", {}))
    v.update(_inference_vars(config, gpus_per_node))
    if nodes == 1:
        v["backend_port"] = v["router_port"]          # a single node serves on the public port itself
    v.update(config_path=str(inference_config), config_dir=str(Path(inference_config).parent), num_nodes=nodes)
    return _render("inference.sbatch.j2", config.slurm, v)
