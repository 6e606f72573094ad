"""Multi-process plumbing on CPU (gloo, world_size 2): data-parallel and expert-parallel RL
steps must reproduce the single-process result."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]

WORKER = r"""
import json, os, sys, torch
sys.path.insert(0, {root!r})
from prime_rl_b200.configs.trainer import TrainerConfig
from prime_rl_b200.trainer.rl.train import RLTrainer
from prime_rl_b200.utils.logger import setup_logger
setup_logger("warning")
torch.manual_seed(0)
cfg = TrainerConfig.model_validate(json.loads({cfg!r}))
tr = RLTrainer(cfg).setup()
out = []
for _ in range(2):
    m = tr.step()
    out.append([m["loss"], m["optim/grad_norm"], m["entropy"]])
with tr.model.full_parameters():
    w = next(p for _, p in tr.model.model.layers[0].named_parameters() if p.dim() == 2).detach().double().clone()
    e = tr.model.model.embed_tokens.weight.detach().double().clone()
res = dict(rank=tr.world.rank, steps=out, wsum=float(w.sum()), wabs=float(w.abs().sum()), esum=float(e.abs().sum()),
           fsdp=getattr(tr.model.layer_hooks, "stats", None), sharded=[bool(g.sharded) for g in tr.optimizer.groups])
open(os.path.join({out!r}, f"rank{{tr.world.rank}}.json"), "w").write(json.dumps(res))
import torch.distributed as dist
if dist.is_initialized():
    dist.barrier(); dist.destroy_process_group()
"""



def _fresh_port() -> int:
    """A port that is free now (a neighbour of a free port is not known to be free)."""
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _run(tmp_path, port, world, cfg):
    port = _fresh_port()
    tag = (f"{world}_{cfg['model'].get('ep', 1)}_{cfg['model'].get('cp', 1)}_{cfg['model'].get('cp_style', 'ring')}"
           f"_z{cfg['model'].get('zero_stage', 2)}_{'ac' if cfg['model'].get('ac') else 'noac'}"
           f"_{cfg.get('optim', {}).get('type', 'adamw')}{int(bool(cfg.get('optim', {}).get('distributed', True)))}")
    script = tmp_path / f"worker_{tag}.py"
    out = tmp_path / f"out_{tag}"
    out.mkdir()
    cfg = dict(cfg, output_dir=str(out))
    script.write_text(WORKER.format(root=str(ROOT), cfg=json.dumps(cfg), out=str(out)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
    if world == 1:
        # one thread, as torchrun gives every rank of the multi-process runs: the reduction order is then fixed
        env.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", OMP_NUM_THREADS="1", MKL_NUM_THREADS="1")
        cmd = [sys.executable, str(script)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.loads((out / f"rank{i}.json").read_text()) for i in range(world)]


BASE = {
    "model": {"name": "tiny-qwen3-moe", "seq_len": 256, "ep": 1, "ac": None, "debug": {"random_init": True}},
    "data": {"fake": {"batch_size": 2}}, "optim": {"lr": 1e-3, "max_norm": 1.0}, "monitors": {"file": None},
}


@pytest.mark.slow
def test_dp2_and_ep2_match_single_process(tmp_path, free_port):
    single = _run(tmp_path, free_port, 1, BASE)[0]
    dp2 = _run(tmp_path, free_port + 1, 2, BASE)
    ep_cfg = json.loads(json.dumps(BASE))
    ep_cfg["model"]["ep"] = 2
    ep2 = _run(tmp_path, free_port + 2, 2, ep_cfg)
    # The fake loader seeds by dp rank, so the 2-rank global batch differs from the 1-rank one;
    # what must hold: ranks agree with each other, and EP == DP on identical data.
    for runs in (dp2, ep2):
        assert runs[0]["wsum"] == pytest.approx(runs[1]["wsum"], rel=1e-9)
        assert runs[0]["steps"][0][1] == pytest.approx(runs[1]["steps"][0][1], rel=1e-6)
    assert dp2[0]["wsum"] == pytest.approx(ep2[0]["wsum"], rel=1e-6)
    assert dp2[0]["wabs"] == pytest.approx(ep2[0]["wabs"], rel=1e-6)
    for a, b in zip(dp2[0]["steps"], ep2[0]["steps"]):
        assert a[0] == pytest.approx(b[0], rel=1e-4, abs=1e-6)
        assert a[1] == pytest.approx(b[1], rel=1e-4)
    assert single["steps"][0][1] > 0


@pytest.mark.slow
@pytest.mark.parametrize("style", ["ring", "ulysses", "ring:ring"])
def test_cp2_matches_single_process(tmp_path, free_port, style):
    """Context-parallel ranks of one replica see the same rows, so CP=2 must reproduce CP=1 ("ring:ring": K / V blocks
    passed rank to rank, partial attention per step merged through the log-sum-exp, dK / dV returned to the owners)."""
    base = json.loads(json.dumps(BASE))
    base["model"]["name"] = "tiny-qwen3"
    single = _run(tmp_path, free_port, 1, base)[0]
    cfg = json.loads(json.dumps(base))
    style, _, exchange = style.partition(":")
    cfg["model"].update(cp=2, cp_style=style)
    if exchange:
        cfg["model"]["cp_kv_exchange"] = exchange
    cp2 = _run(tmp_path, free_port + 1, 2, cfg)
    assert cp2[0]["wsum"] == pytest.approx(cp2[1]["wsum"], rel=1e-9)
    assert cp2[0]["wabs"] == pytest.approx(single["wabs"], rel=1e-5)
    # (the plain sum of a weight matrix is dominated by cancellation: updates of weights whose gradient is at rounding
    # level can flip sign between two runs, so it gets a looser bound than the sum of magnitudes above)
    assert cp2[0]["wsum"] == pytest.approx(single["wsum"], abs=2e-3)
    for a, b in zip(single["steps"], cp2[0]["steps"]):
        assert a[0] == pytest.approx(b[0], rel=1e-3, abs=1e-6)     # loss
        assert a[1] == pytest.approx(b[1], rel=1e-3)               # grad norm
        assert a[2] == pytest.approx(b[2], rel=1e-4)               # entropy


@pytest.mark.slow
@pytest.mark.parametrize("ac", [{"mode": "full", "freq": 1}, None])
def test_parameter_sharding_matches_the_replicated_parameters_run(tmp_path, free_port, ac):
    """ZeRO-3 (every rank keeps half of each layer, layers are gathered as they run, gradients reduce-scattered
    per layer) must give the losses, gradient norms and weights of ZeRO-2 (parameters replicated), with and
    without activation recomputation, and for a dense as well as an MoE + expert-parallel model."""
    for name, ep in (("tiny-qwen3", 1), ("tiny-qwen3-moe", 2)):
        base = json.loads(json.dumps(BASE))
        base["model"].update(name=name, ep=ep, ac=ac)
        z2 = _run(tmp_path, free_port, 2, base)
        cfg = json.loads(json.dumps(base))
        cfg["model"]["zero_stage"] = 3
        z3 = _run(tmp_path, free_port + 1, 2, cfg)
        assert z3[0]["fsdp"] is not None and z3[0]["fsdp"]["gathers"] > 0 and z3[0]["fsdp"]["reduce_scatters"] > 0
        assert z2[0]["fsdp"] is None
        for r in range(2):
            for a, b in zip(z2[r]["steps"], z3[r]["steps"]):
                assert a[0] == pytest.approx(b[0], rel=1e-5, abs=1e-7)       # loss
                assert a[1] == pytest.approx(b[1], rel=1e-4)                  # gradient norm
            assert z2[r]["wsum"] == pytest.approx(z3[r]["wsum"], rel=1e-6, abs=1e-6)
            assert z2[r]["wabs"] == pytest.approx(z3[r]["wabs"], rel=1e-6)
            assert z2[r]["esum"] == pytest.approx(z3[r]["esum"], rel=1e-6)


@pytest.mark.slow
def test_cpu_optimizer_with_gradients_accumulated_on_the_host_matches_the_device_path(tmp_path, free_port):
    """ZeRO-3 with ``full_offload``: every layer's reduced gradient slice is handed to the host accumulator as its
    reduce-scatter completes and the C++ AdamW reads it there; losses, gradient norms and weights must follow the
    run that keeps gradients and optimizer on the device."""
    base = json.loads(json.dumps(BASE))
    base["model"].update(name="tiny-qwen3", ep=1, zero_stage=3)
    base["optim"] = dict(base["optim"], weight_decay=0.01)
    (tmp_path / "dev").mkdir()
    (tmp_path / "host").mkdir()
    dev = _run(tmp_path / "dev", free_port, 2, base)
    cfg = json.loads(json.dumps(base))
    cfg["model"]["full_offload"] = {"chunk_elements": 4096, "max_pinned_slots": 2, "numa_bind": False}
    host = _run(tmp_path / "host", free_port + 1, 2, cfg)
    for r in range(2):
        for a, b in zip(dev[r]["steps"], host[r]["steps"]):
            assert a[0] == pytest.approx(b[0], rel=1e-4, abs=1e-6)
            assert a[1] == pytest.approx(b[1], rel=1e-3)
        assert dev[r]["wabs"] == pytest.approx(host[r]["wabs"], rel=1e-5)
        assert dev[r]["esum"] == pytest.approx(host[r]["esum"], rel=1e-5)


@pytest.mark.slow
def test_muon_with_the_orthogonalisations_dealt_out_matches_every_rank_doing_all(tmp_path, free_port):
    """Two data-parallel ranks: with ``optim.distributed`` the optimizer state is partitioned, the update directions are
    gathered, every matrix is orthogonalised by one rank and the updates return through a reduce-scatter; the weights
    and the losses must be those of the run where both ranks keep whole state and orthogonalise everything."""
    runs = {}
    for i, distributed in enumerate((False, True, "zero3")):
        cfg = json.loads(json.dumps(BASE))
        cfg["model"]["name"] = "tiny-qwen3-moe"
        cfg["optim"] = {"type": "muon", "lr": 1e-3, "max_norm": 1.0, "distributed": bool(distributed)}
        if distributed == "zero3":
            cfg["model"]["zero_stage"] = 3          # parameters sharded per layer as well: the slices are per layer unit
        runs[distributed] = _run(tmp_path, free_port + i, 2, cfg)
    for r in range(2):
        for other in (True, "zero3"):
            a, b = runs[False][r], runs[other][r]
            assert a["wsum"] == pytest.approx(b["wsum"], rel=1e-6, abs=1e-7)
            for x, y in zip(a["steps"], b["steps"]):
                assert x[0] == pytest.approx(y[0], rel=1e-5, abs=1e-7)
    assert runs["zero3"][0]["fsdp"] is not None
    for r in range(2):
        a, b = runs[False][r], runs[True][r]
        assert a["wsum"] == pytest.approx(b["wsum"], rel=1e-6, abs=1e-7)
        assert a["wabs"] == pytest.approx(b["wabs"], rel=1e-6)
        assert a["esum"] == pytest.approx(b["esum"], rel=1e-6)
        for x, y in zip(a["steps"], b["steps"]):
            assert x[0] == pytest.approx(y[0], rel=1e-5, abs=1e-7)
    assert runs[True][0]["wsum"] == pytest.approx(runs[True][1]["wsum"], rel=1e-9)
    # the distributed run partitions master weights and momentum over the ranks, the other keeps them whole everywhere
    assert all(runs[True][0]["sharded"]) and not any(runs[False][0]["sharded"])


@pytest.mark.slow
@pytest.mark.parametrize("name", ["tiny-nemotron-h", "tiny-qwen3.5-moe", "tiny-glm-moe-dsa", "tiny-deepseek-v4"])
def test_cp2_of_the_recurrent_state_families_matches_single_process(tmp_path, free_port, name):
    """Mamba-2 / gated delta-net layers under context parallelism: the sequence split is traded for a head split
    around the convolution and the scan (every rank runs the whole sequence of half of the heads); attention layers
    run the Ulysses exchange. (GLM-MoE-DSA: latent K / V rows and indexer keys gathered whole, local queries select and
    attend over the global sequence.) CP = 2 must reproduce CP = 1."""
    base = json.loads(json.dumps(BASE))
    base["model"]["name"] = name
    single = _run(tmp_path, free_port, 1, base)[0]
    cfg = json.loads(json.dumps(base))
    cfg["model"].update(cp=2, cp_style="ulysses")
    cp2 = _run(tmp_path, free_port + 1, 2, cfg)
    assert cp2[0]["wsum"] == pytest.approx(cp2[1]["wsum"], rel=1e-9)
    assert cp2[0]["esum"] == pytest.approx(single["esum"], rel=1e-5)
    for a, b in zip(single["steps"], cp2[0]["steps"]):
        assert a[0] == pytest.approx(b[0], rel=1e-3, abs=1e-6)     # loss
        assert a[1] == pytest.approx(b[1], rel=2e-3)               # grad norm
        assert a[2] == pytest.approx(b[2], rel=1e-4)               # entropy


SFT_WORKER = r"""
import json, os, sys, torch
sys.path.insert(0, {root!r})
from prime_rl_b200.configs.sft import SFTConfig
from prime_rl_b200.trainer.sft.train import SFTTrainer
from prime_rl_b200.utils.logger import setup_logger
setup_logger("warning")
torch.manual_seed(0)
tr = SFTTrainer(SFTConfig.model_validate(json.loads({cfg!r}))).setup()
out = []
for _ in range(2):
    m = tr.step()
    out.append([m["loss"], m["optim/grad_norm"], m["loss_tokens"]])
w = next(p for _, p in tr.model.model.layers[0].named_parameters() if p.dim() == 2).detach().double()
open(os.path.join({out!r}, f"rank{{tr.world.rank}}.json"), "w").write(json.dumps(dict(steps=out, wsum=float(w.sum()),
                                                                                      wabs=float(w.abs().sum()))))
import torch.distributed as dist
if dist.is_initialized():
    dist.barrier(); dist.destroy_process_group()
"""


def _run_sft(tmp_path, port, world, cfg, tag):
    port = _fresh_port()
    script = tmp_path / f"sft_{tag}.py"
    out = tmp_path / f"sft_out_{tag}"
    out.mkdir()
    cfg = dict(cfg, output_dir=str(out))
    script.write_text(SFT_WORKER.format(root=str(ROOT), cfg=json.dumps(cfg), out=str(out)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
    if world == 1:
        # one thread, as torchrun gives every rank of the multi-process runs: the reduction order is then fixed
        env.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", OMP_NUM_THREADS="1", MKL_NUM_THREADS="1")
        cmd = [sys.executable, str(script)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.loads((out / f"rank{i}.json").read_text()) for i in range(world)]


@pytest.mark.slow
@pytest.mark.parametrize("style,exchange", [("ulysses", "nccl"), ("ring", "ring")])
def test_sft_trainer_with_context_parallelism_matches_single_process(tmp_path, free_port, style, exchange):
    """SFT under context parallelism: the two ranks of the replica read the same packed rows, each runs its chunks and
    sums the loss of its own tokens over the global count of loss tokens; losses and weights equal the single process."""
    base = {"model": {"name": "tiny-qwen3", "ac": None, "debug": {"random_init": True}},
            "data": {"type": "fake", "batch_size": 4, "seq_len": 128, "micro_batch_size": 1, "length": "variable",
                     "input_ids": "random"},
            "optim": {"lr": 1e-3, "max_norm": 1.0}, "monitors": {"file": None}, "max_steps": 2}
    single = _run_sft(tmp_path, free_port, 1, base, "single")[0]
    cfg = json.loads(json.dumps(base))
    cfg["model"].update(cp=2, cp_style=style, cp_kv_exchange=exchange)
    cp2 = _run_sft(tmp_path, free_port + 1, 2, cfg, f"cp2_{style}")
    assert cp2[0]["wsum"] == pytest.approx(cp2[1]["wsum"], rel=1e-9)
    assert cp2[0]["wabs"] == pytest.approx(single["wabs"], rel=1e-5)
    for a, b in zip(single["steps"], cp2[0]["steps"]):
        assert a[2] == b[2]                                         # the same loss tokens
        assert a[0] == pytest.approx(b[0], rel=1e-4, abs=1e-6)      # loss
        assert a[1] == pytest.approx(b[1], rel=1e-3)                # gradient norm
