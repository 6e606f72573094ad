"""fp8 block quantisation helpers and the checkpoint conversion tools (CPU)."""

import json

import torch

from prime_rl_b200.models import build_model, resolve_arch
from prime_rl_b200.models.fp8 import dequantize_fp8_blockwise, quantize_to_fp8_blockwise
from prime_rl_b200.trainer.weights import save_hf_checkpoint


def test_fp8_block_quantiser_round_trip():
    torch.manual_seed(0)
    w = torch.randn(3, 200, 330) * torch.logspace(-2, 1, 330)
    q, s = quantize_to_fp8_blockwise(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 2, 3)
    back = dequantize_fp8_blockwise(q, s, torch.float32)
    # e4m3 has 3 mantissa bits: relative error of a block's largest values <= 2^-4
    blocks_max = w.abs().amax()
    assert (back - w).abs().max() <= blocks_max * 2 ** -4
    assert torch.allclose(s[0, 0, 0], w[0, :128, :128].abs().max() / 448.0)


def test_bf16_fp8_directory_round_trip(tmp_path):
    from prime_rl_b200.tools import convert_bf16_to_fp8, convert_fp8_to_bf16
    from prime_rl_b200.tools._io import read_dir

    model = build_model(resolve_arch("tiny-qwen3-moe"), device="cpu", dtype=torch.bfloat16, seed=0)
    src = save_hf_checkpoint(model, tmp_path / "bf16")
    fp8 = convert_bf16_to_fp8.convert(src, tmp_path / "fp8")
    cfg = json.loads((fp8 / "config.json").read_text())
    assert cfg["quantization_config"]["weight_block_size"] == [128, 128]
    sd8 = read_dir(fp8)
    assert any(k.endswith("_scale_inv") for k in sd8)
    assert any(v.dtype == torch.float8_e4m3fn for v in sd8.values())
    back = convert_fp8_to_bf16.convert(fp8, tmp_path / "bf16_again")
    a, b = read_dir(src), read_dir(back)
    assert set(a) == set(b)
    for k in a:
        err = (a[k].float() - b[k].float()).abs().max()
        assert err <= a[k].float().abs().max() * 2 ** -4 + 1e-6, k
    assert "quantization_config" not in json.loads((back / "config.json").read_text())


def test_dcp_to_bf16(tmp_path):
    from prime_rl_b200.tools import convert_dcp_to_bf16
    from prime_rl_b200.tools._io import read_dir
    from prime_rl_b200.trainer.ckpt import CheckpointManager, Progress

    arch = resolve_arch("tiny-qwen3")
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=1)
    mgr = CheckpointManager(tmp_path, None)
    path = mgr.save(3, model, None, Progress())
    out = convert_dcp_to_bf16.convert(path, tmp_path / "hf", "tiny-qwen3")
    hf = read_dir(out)
    ref = read_dir(save_hf_checkpoint(model, tmp_path / "ref"))
    assert set(hf) == set(ref)
    for k in ref:
        assert torch.equal(hf[k], ref[k]), k


def test_traces_to_parquet(tmp_path):
    import pyarrow.parquet as pq

    from prime_rl_b200.tools import convert_traces_to_hf_dataset as t

    d = tmp_path / "run" / "logs"
    d.mkdir(parents=True)
    rows = [{"env_name": "copy", "task_id": i, "reward": i / 4, "prompt_ids": [1, 2], "completion_ids": [3]} for i in range(5)]
    (d / "traces_orchestrator_000000.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n{bad")
    n = t.convert(tmp_path / "run", tmp_path / "out.parquet", min_reward=0.5)
    assert n == 3
    assert pq.read_table(str(tmp_path / "out.parquet")).num_rows == 3
