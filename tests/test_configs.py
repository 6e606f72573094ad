import json

import pytest

from prime_rl_b200.configs.base import cli
from prime_rl_b200.configs.trainer import TrainerConfig


def test_defaults_and_dotted_flags():
    c = cli(TrainerConfig, ["--model.seq-len", "4096", "--optim.lr", "3e-5", "--max-steps", "7"])
    assert c.model.seq_len == 4096 and c.optim.lr == 3e-5 and c.optim.type == "adamw" and c.max_steps == 7


def test_toml_merge_and_precedence(tmp_path):
    a = tmp_path / "a.toml"
    b = tmp_path / "b.toml"
    a.write_text('max_steps = 5\n[model]\nname = "tiny-qwen3"\nseq_len = 512\n[optim]\nlr = 1e-4\n')
    b.write_text("[model]\nseq_len = 1024\n")
    c = cli(TrainerConfig, ["@", str(a), "@", str(b), "--optim.lr", "2e-4"])
    assert c.model.name == "tiny-qwen3" and c.model.seq_len == 1024 and c.optim.lr == 2e-4 and c.max_steps == 5


def test_bool_none_and_bare_subconfig():
    c = cli(TrainerConfig, ["--model.lora", "--no-model.ac", "--enable-router-replay", "--ckpt.interval", "3",
                            "--model.compile", "None", "--data.fake.batch-size", "4"])
    assert c.model.lora is not None and c.model.lora.rank == 16
    assert c.model.ac is None and c.enable_router_replay is True and c.ckpt.interval == 3
    assert c.model.compile is None
    c2 = cli(TrainerConfig, ["--no-enable-router-replay", "--resume"])
    assert c2.enable_router_replay is False and c2.resume is not None and c2.resume.step is None


def test_discriminated_unions():
    c = cli(TrainerConfig, ["--loss.type", "icepop", "--loss.ratio-high", "4.0", "--scheduler.type", "cosine",
                            "--max-steps", "100", "--weight-broadcast.type", "nccl"])
    assert c.loss.type == "icepop" and c.loss.ratio_high == 4.0 and c.loss.ratio_low == 0.2
    assert c.scheduler.type == "cosine" and c.weight_broadcast.port == 29501


def test_validators():
    with pytest.raises(Exception):
        cli(TrainerConfig, ["--scheduler.type", "cosine"])  # needs max_steps
    with pytest.raises(Exception):
        cli(TrainerConfig, ["--model.lora", "--weight-broadcast.type", "nccl"])
    with pytest.raises(Exception):
        cli(TrainerConfig, ["--env-vars", '{"CUDA_VISIBLE_DEVICES": "0"}'])
    with pytest.raises(Exception):
        cli(TrainerConfig, ["--model.unknown-field", "1"])


def test_resolved_json_round_trip():
    c = cli(TrainerConfig, ["--model.lora.rank", "8", "--max-steps", "3"])
    again = TrainerConfig.model_validate(json.loads(c.to_json()))
    assert again == c


def test_tensor_parallel_inference_in_the_rl_config(tmp_path):
    """num_infer_gpus splits into replicas x tensor-parallel ranks; sharded engines only take filesystem updates."""
    import pytest

    from prime_rl_b200.configs.rl import RLConfig

    base = {"deployment": {"type": "single_node", "num_infer_gpus": 4, "num_train_gpus": 2},
            "inference": {"vllm": {"tensor_parallel_size": 2}}, "output_dir": str(tmp_path)}
    cfg = RLConfig.model_validate(base)
    assert cfg.inference.vllm.data_parallel_size == 2 and cfg.inference.vllm.tensor_parallel_size == 2
    with pytest.raises(ValueError):
        RLConfig.model_validate(dict(base, deployment=dict(base["deployment"], num_infer_gpus=3)))
    with pytest.raises(ValueError):
        RLConfig.model_validate(dict(base, trainer={"weight_broadcast": {"type": "nccl"}}))
