import pytest
import torch

from prime_rl_b200.configs.trainer import (AdamWConfig, CheckpointConfig, CosineSchedulerConfig, LinearSchedulerConfig,
                                           MuonConfig, SGDConfig, SignSGDConfig, TrainerConfig)
from prime_rl_b200.models import build_model, resolve_arch
from prime_rl_b200.trainer.ckpt import CheckpointManager, Progress
from prime_rl_b200.trainer.optim import LRSchedule, setup_optimizer
from prime_rl_b200.trainer.rl.train import RLTrainer
from prime_rl_b200.trainer.weights import load_hf_checkpoint, save_hf_checkpoint


def _model(seed=0):
    return build_model(resolve_arch("tiny-qwen3-moe"), device="cpu", dtype=torch.float32, seed=seed)


def test_flat_adamw_matches_torch():
    m1, m2 = _model(), _model()
    opt = setup_optimizer(AdamWConfig(lr=1e-3, weight_decay=0.1, max_norm=None), m1)
    ref = torch.optim.AdamW(m2.parameters(), lr=1e-3, weight_decay=0.1, betas=(0.9, 0.999), eps=1e-8)
    for step in range(3):
        g = torch.Generator().manual_seed(step)
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            grad = torch.randn(p1.shape, generator=g)
            p1.grad = grad.clone()
            p2.grad = grad.clone()
        opt.buf.accumulate_grads()
        opt.step()
        opt.zero_grad()
        ref.step()
    for (n, p1), p2 in zip(m1.named_parameters(), m2.parameters()):
        assert torch.allclose(p1, p2, atol=1e-6), n


def test_clipping_and_other_optimizers():
    for cfg in (SGDConfig(lr=1e-2, max_norm=1.0), SignSGDConfig(lr=1e-3, max_norm=1.0), MuonConfig(lr=1e-3, max_norm=1.0)):
        m = _model()
        before = [p.detach().clone() for p in m.parameters()]
        opt = setup_optimizer(cfg, m)
        for p in m.parameters():
            p.grad = torch.ones_like(p) * 10
        opt.buf.accumulate_grads()
        norm = opt.step()
        assert float(norm) > 1.0 and torch.isfinite(norm)
        assert any(not torch.equal(a, b) for a, b in zip(before, m.parameters()))
        assert all(torch.isfinite(p).all() for p in m.parameters())


def test_lr_schedules():
    lin = LRSchedule(LinearSchedulerConfig(warmup_steps=2, decay_steps=4, min_lr=0.0), 10, 1.0)
    assert lin.lr_at(0) < lin.lr_at(1) < lin.lr_at(2) == 1.0 and lin.lr_at(5) == 1.0
    assert lin.lr_at(6) == 1.0 and lin.lr_at(7) < 1.0 and lin.lr_at(9) < lin.lr_at(8)
    cos = LRSchedule(CosineSchedulerConfig(warmup_steps=2, min_lr=0.1), 12, 1.0)
    assert cos.lr_at(2) == 1.0 and abs(cos.lr_at(12) - 0.1) < 1e-9 and cos.lr_at(7) < cos.lr_at(3)


def test_dcp_checkpoint_round_trip_uses_prime_names(tmp_path):
    m = _model()
    opt = setup_optimizer(AdamWConfig(lr=1e-3), m)
    for p in m.parameters():
        p.grad = torch.randn_like(p)
    opt.buf.accumulate_grads()
    opt.step()
    mgr = CheckpointManager(tmp_path, CheckpointConfig(interval=1))
    mgr.save(4, m, opt, Progress(step=4, total_tokens=123, total_samples=7))
    assert (tmp_path / "checkpoints" / "step_4" / "trainer" / ".metadata").exists()
    m2 = _model(seed=1)
    opt2 = setup_optimizer(AdamWConfig(lr=1e-3), m2)
    prog = Progress()
    mgr.load(4, m2, opt2, prog)
    assert prog.total_tokens == 123 and opt2.step_count == 1
    for (n, a), b in zip(m.named_parameters(), m2.parameters()):
        assert torch.equal(a, b), n
    assert torch.equal(opt.groups[0].exp_avg, opt2.groups[0].exp_avg)
    import torch.distributed.checkpoint as dcp
    keys = dcp.FileSystemReader(str(mgr.step_path(4))).read_metadata().state_dict_metadata.keys()
    assert "app.model.model.layers.0.self_attn.q_proj.weight" in keys          # canonical, unfused
    assert "app.model.model.layers.0.mlp.experts.gate_proj" in keys
    assert not any("qkv_proj" in k or "gate_up_proj" in k for k in keys)


def test_retention(tmp_path):
    m = _model()
    mgr = CheckpointManager(tmp_path, CheckpointConfig(interval=1, keep_last=2, keep_interval=4))
    for s in range(1, 7):
        mgr.save(s, m, None, Progress(step=s))
        mgr.maybe_clean()
    left = sorted(int(p.name.split("_")[1]) for p in (tmp_path / "checkpoints").iterdir())
    assert left == [4, 5, 6]


def test_hf_export_import(tmp_path):
    m = _model()
    save_hf_checkpoint(m, tmp_path / "hf", max_shard_bytes=200_000, dtype=torch.float32)
    files = list((tmp_path / "hf").glob("*.safetensors"))
    assert len(files) > 1 and (tmp_path / "hf" / "model.safetensors.index.json").exists()
    m2 = _model(seed=3)
    load_hf_checkpoint(m2, tmp_path / "hf")
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)


def test_trainer_resume_continues_identically(tmp_path):
    base = {"model": {"name": "tiny-qwen3", "seq_len": 128, "ac": None, "debug": {"random_init": True}},
            "data": {"fake": {"batch_size": 2}}, "optim": {"lr": 1e-3}, "monitors": {"file": None}}
    full = TrainerConfig.model_validate(dict(base, max_steps=4, output_dir=str(tmp_path / "a")))
    t = RLTrainer(full, device=torch.device("cpu")).setup()
    losses = [t.step()["loss"] for _ in range(4)]
    part = TrainerConfig.model_validate(dict(base, max_steps=2, output_dir=str(tmp_path / "b"), ckpt={"interval": 2}))
    RLTrainer(part, device=torch.device("cpu")).setup().run()
    res = TrainerConfig.model_validate(dict(base, max_steps=4, output_dir=str(tmp_path / "b"), ckpt={"interval": 2},
                                            resume={}))
    t2 = RLTrainer(res, device=torch.device("cpu")).setup()
    assert t2.progress.step == 2
    resumed = [t2.step()["loss"] for _ in range(2)]
    assert resumed == [pytest_approx(x) for x in losses[2:]]


def pytest_approx(x):
    import pytest
    return pytest.approx(x, rel=1e-5, abs=1e-7)


@pytest.mark.parametrize("mode", ["state", "cpu"])
def test_optimizer_offload_matches_device_resident_step(mode):
    """Optimizer state parked in host memory (and the C++ CPU update) give the same parameters
    as the resident optimizer."""
    import copy

    from prime_rl_b200.configs.trainer import AdamWConfig
    from prime_rl_b200.trainer.optim import FlatOptimizer

    torch.manual_seed(0)
    ref_model = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Linear(40, 8))
    off_model = copy.deepcopy(ref_model)
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1, max_norm=0.5)
    opt_ref = FlatOptimizer(cfg, list(ref_model.named_parameters()))
    opt_off = FlatOptimizer(cfg, list(off_model.named_parameters()), offload=mode, offload_chunk=300)
    for step in range(3):
        x = torch.randn(16, 24)
        for model, opt in ((ref_model, opt_ref), (off_model, opt_off)):
            opt.zero_grad()
            model(x).pow(2).mean().backward()
            opt.reduce_gradients()
            opt.step()
    for a, b in zip(ref_model.parameters(), off_model.parameters()):
        assert torch.allclose(a, b, rtol=2e-5, atol=2e-6)
    sd = opt_off.state_dict()
    assert set(sd["state"]) >= {"exp_avg", "exp_avg_sq"}


def test_gradient_offload_accumulates_pieces_on_the_host_with_bounded_slots():
    """Pieces of a gradient shard submitted while 'the backward pass goes on' end up summed in the host
    accumulator; more pieces than pinned slots only cause waiting, never loss; bf16 sources take the C++ path."""
    import torch

    from prime_rl_b200.trainer.optim_offload import GradientOffload

    torch.manual_seed(0)
    n = 10_000
    go = GradientOffload(n, torch.device("cpu"), chunk_elements=1024, max_pinned_slots=2)
    total = torch.zeros(n)
    for _ in range(3):                                   # three micro-batches
        g = torch.randn(n)
        total += g
        for lo in range(0, n, 2500):                     # four layers' slices each
            piece = g[lo:lo + 2500].clone()
            go.submit(piece, offset=lo)
            assert float(piece.abs().sum()) == 0.0       # the device copy is cleared for the next micro-batch
    acc = go.wait()
    assert torch.allclose(acc, total, atol=1e-5) and go.stats["pieces"] == 3 * 4 * 3
    go.reset()
    assert float(go.wait().abs().sum()) == 0.0
    go.close()
    gb = GradientOffload(512, torch.device("cpu"), chunk_elements=512, src_dtype=torch.bfloat16)
    src = torch.randn(512).bfloat16()
    gb.submit_at(0, src.clone())
    gb.submit_at(0, src.clone())
    assert torch.allclose(gb.wait(), 2 * src.float(), atol=1e-6)
    gb.close()


def test_numa_binding_reads_the_gpu_node_from_sysfs(tmp_path):
    import os

    from prime_rl_b200.trainer.optim_offload import bind_to_gpu_numa_node, cpus_of_numa_node, numa_node_of_gpu

    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    mine = sorted(os.sched_getaffinity(0))
    (node / "cpulist").write_text(f"{mine[0]},{mine[-1]}-{mine[-1]},9999\n")
    assert numa_node_of_gpu("00000000:1B:00.0", str(tmp_path)) == 1          # CUDA's 8-digit domain form
    assert cpus_of_numa_node(1, str(tmp_path)) == {mine[0], mine[-1], 9999}
    calls = []
    assert bind_to_gpu_numa_node("0000:1b:00.0", str(tmp_path), setaffinity=lambda pid, c: calls.append((pid, c))) == 1
    assert calls == [(0, {mine[0], mine[-1]})]                               # only cores this process may use
    (dev / "numa_node").write_text("-1\n")
    assert bind_to_gpu_numa_node("0000:1b:00.0", str(tmp_path), setaffinity=lambda *a: calls.append(a)) is None
    assert len(calls) == 1 and numa_node_of_gpu("0000:ff:00.0", str(tmp_path)) is None
