"""Peer-memory expert-parallel dispatcher against the all-to-all baseline on two GPUs
(child processes, one per GPU; NVLS off, plain peer loads / stores only)."""

import os
import subprocess
import sys

from pathlib import Path

import pytest
import torch

ROOT = str(Path(__file__).resolve().parents[1])      # the children are run as `-m tests.distributed.<name>`

pytestmark = pytest.mark.gpu


def test_p2p_dispatcher_matches_all_to_all():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", EP_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", "-m", "tests.distributed.ep_dispatch"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "EP_SELFTEST_OK" in out.stdout and "EP_FP8_PAYLOAD_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_gemm_reduce_scatter_over_peer_memory():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", FUSED_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29534", "-m", "tests.distributed.fused_collectives"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "FUSED_RS_OK" in out.stdout and "FUSED_AG_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_weight_push_over_peer_memory():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", P2P_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29535", "-m", "tests.distributed.weight_push"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "P2P_WEIGHTS_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_all_to_all_over_peer_memory():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", P2P_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29536", "-m", "tests.distributed.p2p_a2a"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "P2P_A2A_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_bounded_peer_wait_reports_timeout_instead_of_hanging():
    """A wait on a flag that nothing sets runs out (about 2 s of GPU time), records
    kTimeoutPeerFlag in the status word and returns; the context stays usable."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.ops import _runtime as rt

    dev = torch.device("cuda", 0)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    st = rt.status_tensor(dev)
    st.zero_()
    rc = rt.lib().prb_ep_wait(flags.data_ptr(), 2, 0, 1, st.data_ptr(), rt.stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 5            # kTimeoutPeerFlag
    with pytest.raises(Exception):
        rt.check_status()
    st.zero_()
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0      # the device still answers


def test_trainer_step_with_peer_memory_expert_parallelism():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29537", "-m", "tests.distributed.ep_trainer"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "EP_TRAINER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_context_parallel_attention_with_in_kernel_kv_gather():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", CP_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29538", "-m", "tests.distributed.cp_attention"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "CP_FUSED_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_ring_attention_with_log_sum_exp_merging():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", CP_SELFTEST_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29543", "-m", "tests.distributed.ring_attention"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "RING_ATTN_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_sharded_optimizer_with_peer_memory_collectives():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", P2P_ZERO_TIMING="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29539", "-m", "tests.distributed.zero_collectives"]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "P2P_ZERO_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_tensor_parallel_engine_with_fused_reduce_kernel():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for port, extra in ((29541, []), (29540, ["--cuda-graphs"]), (29544, ["--cuda-graphs", "--expert-parallel"])):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(port), "-m", "tests.distributed.tp_engine", *extra]
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert out.returncode == 0 and "TP_SELFTEST_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
