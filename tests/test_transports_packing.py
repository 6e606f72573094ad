import asyncio
import threading
import time

import pytest
import torch

from prime_rl_b200.configs.algorithm import GRPOAlgoConfig, MaxRLAlgoConfig, RAEAlgoConfig, SFTAlgoConfig
from prime_rl_b200.configs.shared import ZMQTransportConfig
from prime_rl_b200.orchestrator.algo import setup_algorithm
from prime_rl_b200.orchestrator.concurrency import ConcurrencyController
from prime_rl_b200.orchestrator.types import Rollout, Turn
from prime_rl_b200.trainer import batch as B
from prime_rl_b200.transports.batch import (FileSystemBatchReceiver, FileSystemBatchSender, ZMQBatchReceiver,
                                            ZMQBatchSender, micro_batch_to_tensors)
from prime_rl_b200.transports.batch.types import TrainingSample, decode_micro_batches, encode_micro_batches


def _sample(n, env="e", adv=0.5):
    return TrainingSample(token_ids=list(range(n)), mask=[i >= n // 2 for i in range(n)], logprobs=[-0.1] * n,
                          temperatures=[1.0] * n, env_name=env, advantages=[adv] * n, trace_id=f"t{n}", branch_index=0)


def test_ffd_and_balance():
    bins = B.first_fit_decreasing([60, 50, 40, 30, 20, 10], 100)
    assert all(sum([60, 50, 40, 30, 20, 10][i] for i in b) <= 100 for b in bins) and len(bins) == 3
    assign = B.balance([10, 9, 8, 7, 1, 1, 1, 1], 2)
    loads = [sum([10, 9, 8, 7, 1, 1, 1, 1][i] for i in a) for a in assign]
    assert abs(loads[0] - loads[1]) <= 1 and all(len(a) == 4 for a in assign)
    assert B.bin_cost([8192]) > 2 * B.bin_cost([4096])          # quadratic attention term


def test_prepare_batch_grid_alignment_and_dummies():
    samples = [_sample(n) for n in (100, 90, 60, 30, 20)]
    grid = B.prepare_batch(samples, seq_len=128, num_train_workers=2, pad_to_multiple_of=8)
    assert len(grid) == 2 and len(grid[0]) == len(grid[1])          # equal micro-steps (dummy rows fill up)
    seen = 0
    for row in (mb for rank in grid for mb in rank):
        n = len(row.input_ids)
        assert n % 8 == 0 and n <= 128 and sum(row.sequence_lengths) == n
        assert len(row.loss_mask) == len(row.advantages) == len(row.position_ids) == n
        seen += sum(row.loss_mask)
    assert seen == sum(sum(s.mask) for s in samples)
    t = micro_batch_to_tensors(grid[0][0])
    assert t.input_ids.dtype == torch.long and t.position_ids[0] == 0 and t.loss_mask.dtype == torch.bool
    with pytest.raises(ValueError):
        B.prepare_sample(TrainingSample([1, 2], [True, True], [0.0], [1.0, 1.0], "e"), 8)   # misaligned stream


def test_wire_format_round_trip_and_truncation():
    grid = B.prepare_batch([_sample(300)], seq_len=128, num_train_workers=1)
    mb = decode_micro_batches(encode_micro_batches(grid[0]))[0]
    assert len(mb.input_ids) == 128 and mb.trace_ids == ["t300"] and mb.env_names == ["e"]


def test_filesystem_transport(tmp_path):
    grid = B.prepare_batch([_sample(40), _sample(50)], seq_len=64, num_train_workers=2)
    FileSystemBatchSender(tmp_path).send(3, grid)
    assert not list((tmp_path / "batches" / "step_3").glob("*.tmp"))
    r = FileSystemBatchReceiver(tmp_path, dp_rank=1, start_step=3, timeout=5)
    got = r.receive()
    assert [m.input_ids for m in got] == [m.input_ids for m in grid[1]] and r.step == 4
    with pytest.raises(TimeoutError):
        FileSystemBatchReceiver(tmp_path, 0, 9, timeout=0.2).wait()      # a batch that never arrives


def test_zmq_transport(free_port):
    cfg = ZMQTransportConfig(host="127.0.0.1", port=free_port)
    grid = B.prepare_batch([_sample(40), _sample(50)], seq_len=64, num_train_workers=2)
    sender = ZMQBatchSender(cfg, num_ranks=2, ready_timeout=20)
    out = {}

    def recv(rank):
        r = ZMQBatchReceiver(cfg, rank)
        out[rank] = r.receive()
        r.close()

    ths = [threading.Thread(target=recv, args=(i,)) for i in range(2)]
    for t in ths:
        t.start()
    sender.send(0, grid)
    for t in ths:
        t.join(timeout=20)
    sender.close()
    assert [m.input_ids for m in out[0]] == [m.input_ids for m in grid[0]]
    assert [m.input_ids for m in out[1]] == [m.input_ids for m in grid[1]]


def _rollout(reward, n_out=4, gid="g", agent=None):
    t = Turn(prompt_ids=[1, 2, 3], completion_ids=list(range(10, 10 + n_out)), completion_logprobs=[-0.5] * n_out)
    return Rollout(env_name="e", task_id=0, group_id=gid, turns=[t], reward=reward, agent=agent)


def test_algorithms():
    run = asyncio.run
    g = [_rollout(r) for r in (1.0, 0.0, 0.0, 1.0)]
    run(setup_algorithm(GRPOAlgoConfig()).score_group(g))
    assert [r.advantage for r in g] == [0.5, -0.5, -0.5, 0.5]
    g = [_rollout(r) for r in (1.0, 0.0, 0.0, 0.0)]
    run(setup_algorithm(MaxRLAlgoConfig()).score_group(g))
    assert g[0].advantage == pytest.approx(3.0) and g[1].advantage == pytest.approx(-1.0)
    rae = setup_algorithm(RAEAlgoConfig(decay=0.5))
    a, b = _rollout(1.0), _rollout(0.0)
    run(rae.score_group([a]))
    run(rae.score_group([b]))
    assert a.advantage == 0.0 and b.advantage == -1.0 and rae.baselines["e/agent"] == 0.5
    algo = setup_algorithm(GRPOAlgoConfig())
    g[0].advantage = 0.25
    s = algo.to_samples(g[0])[0]
    assert s.mask == [False] * 3 + [True] * 4 and s.advantages[3:] == [0.25] * 4 and s.logprobs[:3] == [0.0] * 3
    sft = setup_algorithm(SFTAlgoConfig()).to_samples(g[0])[0]
    assert sft.ce_weights == [0.0] * 3 + [1.0] * 4 and sft.rl_weights == [0.0] * 7


def test_concurrency_controller():
    from prime_rl_b200.configs.orchestrator import ConcurrencyConfig
    c = ConcurrencyController(ConcurrencyConfig(initial_inflight=8, min_inflight=2, max_inflight=64))
    for _ in range(8):
        c.on_episode_done()
    assert c.update(kv_usage=0.3, inflight=8).limit == 10             # grow x1.25
    assert c.update(kv_usage=0.7, inflight=10).reason == "hold"
    d = c.update(kv_usage=0.85, inflight=10)
    assert d.reason == "soft_trim" and d.limit < 10
    d = c.update(kv_usage=0.95, inflight=8)
    assert d.reason == "hard_trim" and d.cancel == 8 - d.limit
    d = c.update(kv_usage=0.5, preemptions_total=3, inflight=4)
    assert d.reason == "hard_trim" and d.limit >= 2
