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
    """num_infer_gpus splits into replicas x tensor-parallel ranks; every rank of a sharded engine is one
    worker of the in-memory weight transport."""
    import pytest

    from prime_rl_b200.configs.rl import RLConfig

    base = {"deployment": {"type": "single_node", "num_infer_gpus": 4, "num_train_gpus": 2},
            "inference": {"vllm": {"tensor_parallel_size": 2}}, "output_dir": str(tmp_path)}
    cfg = RLConfig.model_validate(base)
    assert cfg.inference.vllm.data_parallel_size == 2 and cfg.inference.vllm.tensor_parallel_size == 2
    with pytest.raises(ValueError):
        RLConfig.model_validate(dict(base, deployment=dict(base["deployment"], num_infer_gpus=3)))
    assert cfg.weight_broadcast.type == "nccl" and cfg.trainer.weight_broadcast.inference_world_size == 4
    assert cfg.orchestrator.weight_broadcast.inference_world_size == 4 and cfg.orchestrator.num_train_workers == 2
    fs = RLConfig.model_validate(dict(base, weight_broadcast={"type": "filesystem"}))
    assert fs.trainer.weight_broadcast.type == fs.orchestrator.weight_broadcast.type == "filesystem"
    assert fs.inference.weight_broadcast.type == "filesystem"


# ---------------------------------------------------------------------- the reference's shipped configs
# ``tests/data/reference_configs/*.json`` hold the parsed key / value trees of every TOML file the reference
# ships under configs/, examples/ and k8s/ (values only, no comments). Each must load into at least one of
# the config classes, as in the reference's own test (tests/unit/test_configs.py:43-53).
import pathlib

import pytest

_REF = sorted((pathlib.Path(__file__).parent / "data" / "reference_configs").glob("*.json"))


def _config_classes():
    from prime_rl_b200.configs.evals import EnvServerConfig, EvalsConfig
    from prime_rl_b200.configs.inference import InferenceConfig
    from prime_rl_b200.configs.orchestrator import OrchestratorConfig
    from prime_rl_b200.configs.rl import RLConfig
    from prime_rl_b200.configs.sft import SFTConfig

    return [RLConfig, SFTConfig, TrainerConfig, OrchestratorConfig, InferenceConfig, EnvServerConfig, EvalsConfig]


def _load(path):
    from pydantic import ValidationError

    tree = json.loads(path.read_text())["config"]
    errors = {}
    for cls in _config_classes():
        try:
            return cls, cls.model_validate(json.loads(json.dumps(tree))), errors
        except (ValidationError, ValueError) as e:
            errors[cls.__name__] = str(e)[:300]
    return None, None, errors


@pytest.mark.parametrize("path", _REF, ids=lambda p: p.stem)
def test_reference_config_file_loads(path):
    cls, cfg, errors = _load(path)
    assert cfg is not None, f"{path.stem}: no config class accepts it: {errors}"


def test_reference_rl_configs_resolve_like_the_reference_launcher():
    """The derived fields of every shipped ``rl`` config follow the launcher's rules: one weight-transfer
    worker per inference GPU (dp x tp), one batch slot per data replica (train GPUs / cp), packing padded to
    cp, NCCL when an inference block is present and no adapters are trained, files otherwise."""
    from prime_rl_b200.configs.rl import RLConfig

    seen = 0
    for path in _REF:
        cls, cfg, _ = _load(path)
        if cls is not RLConfig:
            continue
        seen += 1
        raw = json.loads(path.read_text())["config"]
        t, o, i, d = cfg.trainer, cfg.orchestrator, cfg.inference, cfg.deployment
        assert t.weight_broadcast.type == o.weight_broadcast.type == cfg.weight_broadcast.type
        if "weight_broadcast" not in raw and "weight_broadcast" not in raw.get("trainer", {}) \
                and "weight_broadcast" not in raw.get("orchestrator", {}):
            want = "filesystem" if (t.model.lora is not None or i is None) else "nccl"
            assert cfg.weight_broadcast.type == want, path.stem
        assert o.pad_to_multiple_of == max(1, t.model.cp)
        assert o.seq_len == t.model.seq_len
        if d.type == "single_node":
            if d.num_train_gpus > 1:
                assert o.num_train_workers == d.num_train_gpus // t.model.cp, path.stem
            if i is not None:
                assert i.vllm.data_parallel_size * i.vllm.tensor_parallel_size == d.num_infer_gpus, path.stem
                if hasattr(t.weight_broadcast, "inference_world_size"):
                    assert t.weight_broadcast.inference_world_size == d.num_infer_gpus
                    assert o.weight_broadcast.inference_world_size == d.num_infer_gpus
        else:
            assert o.num_train_workers == d.num_train_nodes * d.gpus_per_node // t.model.cp
        if t.model.lora is not None:
            assert o.model.lora is not None and o.model.lora.rank == t.model.lora.rank
            if i is not None:
                assert i.vllm.enable_lora and i.vllm.max_lora_rank == t.model.lora.rank
        if i is not None:
            assert i.weight_broadcast.type == cfg.weight_broadcast.type
            assert i.output_dir == t.output_dir == o.output_dir
    assert seen >= 35
