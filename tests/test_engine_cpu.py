import json

import pytest
import torch

from prime_rl_b200.engine.engine import Engine
from prime_rl_b200.engine.sampler import SamplingParams, sample
from prime_rl_b200.models import SeqInfo, build_model, resolve_arch


def _engine(name="tiny-qwen3", **kw):
    arch = resolve_arch(name)
    model = build_model(arch, device="cpu", dtype=torch.float32)
    return arch, model, Engine(model, num_pages=256, page_size=16, **kw)


def _greedy_reference(model, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        ids = torch.tensor(toks)
        h = model(ids, SeqInfo.from_lengths([len(toks)], "cpu"))
        toks.append(int(model.logits(h[-1:]).argmax(-1)))
    return toks[len(prompt):]


def test_greedy_decode_matches_uncached_forward():
    arch, model, eng = _engine()
    prompts = [torch.randint(0, arch.vocab_size, (n,)).tolist() for n in (5, 23, 40)]
    reqs = eng.generate_sync(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, r in zip(prompts, reqs):
        assert r.output == _greedy_reference(model, p, 12)
        assert r.finish_reason == "length" and len(r.logprobs) == 12
    assert eng.cache.blocks.num_free + len(eng.cache.blocks.prefix_cache) == 256


def test_prefix_sharing_and_salt():
    arch, model, eng = _engine()
    prompt = torch.randint(0, arch.vocab_size, (50,)).tolist()
    sp = SamplingParams(max_tokens=4, temperature=0.0)
    a = eng.generate_sync([prompt], sp, cache_salt="1")[0]
    hits0 = eng.stats["prefix_hits"]
    b = eng.generate_sync([prompt] * 3, sp, cache_salt="1")
    assert eng.stats["prefix_hits"] - hits0 == 3 * 48          # 3 full pages of 16 tokens each
    assert all(r.output == a.output for r in b)
    hits1 = eng.stats["prefix_hits"]
    eng.generate_sync([prompt], sp, cache_salt="2")            # new policy version: no reuse
    assert eng.stats["prefix_hits"] == hits1


def test_moe_engine_returns_routed_experts_and_logprobs():
    arch, model, eng = _engine("tiny-qwen3-moe")
    eng.runner.capture_routed = True
    prompt = torch.randint(0, arch.vocab_size, (20,)).tolist()
    r = eng.generate_sync([prompt], SamplingParams(max_tokens=5, temperature=1.0, seed=3,
                                                   return_routed_experts=True))[0]
    assert len(r.routed) == 5 and r.routed[0].shape == (arch.num_hidden_layers, arch.num_experts_per_tok)
    assert all(lp <= 0 for lp in r.logprobs)
    # the reported logprob is the model's log-probability of the sampled token
    ids = torch.tensor(prompt + r.output)
    h = model(ids, SeqInfo.from_lengths([len(ids)], "cpu"))
    lp = torch.log_softmax(model.logits(h).float(), -1)
    for i, tok in enumerate(r.output):
        assert abs(float(lp[len(prompt) - 1 + i, tok]) - r.logprobs[i]) < 1e-3


def test_sampler_truncation_and_mask():
    logits = torch.tensor([[5.0, 4.0, 1.0, 0.0, -1.0]] * 2)
    tok, lp, masks = sample(logits, torch.tensor([1.0, 1.0]), torch.tensor([2, -1]), torch.tensor([1.0, 0.6]),
                            want_mask=True)
    assert set(masks[0].tolist()) == {0, 1} and int(tok[0]) in (0, 1)
    assert masks[1].tolist() == [0]                 # top-p 0.6 keeps only the 0.72 head
    assert abs(float(lp[1])) < 1e-6                 # renormalised over the kept set
    g_tok, _, _ = sample(logits, torch.tensor([0.0, 0.0]), torch.tensor([-1, -1]), torch.tensor([1.0, 1.0]))
    assert g_tok.tolist() == [0, 0]


def test_pause_blocks_progress_and_resume_continues():
    import time
    arch, model, eng = _engine()
    eng.start()
    eng.pause()
    req = eng.submit(__import__("prime_rl_b200.engine.engine", fromlist=["Request"]).Request(
        prompt=[1, 2, 3], params=SamplingParams(max_tokens=3, temperature=0.0)))
    time.sleep(0.2)
    assert req.finish_reason is None and not req.output
    eng.resume()
    t0 = time.time()
    while req.finish_reason is None and time.time() - t0 < 20:
        time.sleep(0.01)
    assert req.finish_reason == "length"
    eng.shutdown()


def test_router_places_sessions_and_fans_out_admin_calls():
    """Two CPU engines behind the router: a session always meets the same replica, free requests
    spread, admin calls reach both, metrics are summed."""
    import asyncio

    import httpx

    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.engine.router import HashRing, Router, build_app as build_router, merge_metrics
    from prime_rl_b200.engine.server import build_app
    from prime_rl_b200.models import build_model, resolve_arch

    arch = resolve_arch("tiny-qwen3")
    engines = [Engine(build_model(arch, device="cpu", dtype=torch.float32, seed=3), num_pages=128).start() for _ in range(2)]
    apps = [build_app(e, "tiny-qwen3") for e in engines]
    router = Router(["http://r0", "http://r1"], transports=[httpx.ASGITransport(app=a) for a in apps])
    app = build_router(router)

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://router") as c:
            assert (await c.get("/health")).json()["replicas"] == 2
            body = {"token_ids": [1, 2, 3, 4], "sampling_params": {"max_tokens": 3, "temperature": 0.0}}
            outs = [await c.post("/inference/v1/generate", json=dict(body, cache_salt="conversation-7")) for _ in range(4)]
            assert all(o.status_code == 200 for o in outs)
            served_after_session = list(router.served)
            assert sorted(served_after_session) == [0, 4]                     # one replica took the whole session
            outs = await asyncio.gather(*[c.post("/inference/v1/generate", json=body) for _ in range(6)])
            assert all(o.status_code == 200 for o in outs)
            assert min(router.served) >= 2                                    # the free requests were spread
            texts = {json.dumps(o.json().get("choices", o.json())[0] if "choices" in o.json() else o.json(), sort_keys=True)
                     for o in outs}
            assert len(texts) >= 1
            r = await c.post("/pause")
            assert r.status_code == 200 and r.json()["replicas"] == 2
            assert all(e.paused for e in engines)
            assert (await c.post("/resume")).status_code == 200 and not any(e.paused for e in engines)
            m = (await c.get("/metrics")).text
            assert "vllm:num_requests_running" in m or "num_requests" in m
            st = (await c.get("/router/state")).json()
            assert st["inflight"] == [0, 0] and sum(st["served"]) == 10

    try:
        asyncio.run(go())
    finally:
        for e in engines:
            e.shutdown()
    ring = HashRing([0, 1, 2])
    assert {ring.node(f"k{i}") for i in range(200)} == {0, 1, 2}
    moved = sum(HashRing([0, 1]).node(f"k{i}") != ring.node(f"k{i}") for i in range(200) if ring.node(f"k{i}") != 2)
    assert moved == 0                                                         # only the removed node's keys move
    assert merge_metrics(["# HELP a x\na 1\nb{l=\"1\"} 2\n", "# HELP a x\na 3\n"]) == "# HELP a x\na 4.0\nb{l=\"1\"} 2.0\n"


def test_tensor_parallel_shards_sum_to_the_full_layer():
    """Head-split attention projections and width-split MLP / experts: the sum of the ranks' partial
    outputs is the unsharded output (checked on the projection algebra of one layer)."""
    from prime_rl_b200.engine.tp import shard_tensor
    from prime_rl_b200.models import ModelArch

    arch = ModelArch(model_type="qwen3_moe", hidden_size=64, num_hidden_layers=1, num_attention_heads=8,
                     num_key_value_heads=4, head_dim=16, intermediate_size=96, num_experts=4, num_experts_per_tok=2,
                     moe_intermediate_size=48, vocab_size=128)
    torch.manual_seed(0)
    H, D, nq, nkv, I, E = 64, 16, 8, 4, 48, 4
    qkv = torch.randn((nq + 2 * nkv) * D, H)
    o = torch.randn(H, nq * D)
    gu, down = torch.randn(E, 2 * I, H), torch.randn(E, H, I)
    x = torch.randn(5, H)
    R = 2
    # attention: per-head outputs only depend on the rank's own heads, so o_proj partials add up
    full_heads = (x @ qkv.t())[:, : nq * D]                                  # stand-in for the attention output
    total = torch.zeros(5, H)
    for r in range(R):
        w = shard_tensor("model.layers.0.self_attn.qkv_proj.weight", qkv, arch, r, R)
        assert w.shape == ((nq + 2 * nkv) * D // R, H)
        q_r = (x @ w.t())[:, : nq * D // R]
        torch.testing.assert_close(q_r, full_heads[:, r * nq * D // R:(r + 1) * nq * D // R])
        k_r = (x @ w.t())[:, nq * D // R: (nq + nkv) * D // R]
        torch.testing.assert_close(k_r, (x @ qkv.t())[:, nq * D + r * nkv * D // R: nq * D + (r + 1) * nkv * D // R])
        total += q_r @ shard_tensor("model.layers.0.self_attn.o_proj.weight", o, arch, r, R).t()
    torch.testing.assert_close(total, full_heads @ o.t(), atol=1e-4, rtol=1e-4)
    # experts: silu(gate) * up is elementwise in the intermediate width
    def expert(g_u, dn, e):
        h = x @ g_u[e].t()
        half = h.shape[1] // 2
        return (torch.nn.functional.silu(h[:, :half]) * h[:, half:]) @ dn[e].t()
    for e in range(E):
        parts = sum(expert(shard_tensor("model.layers.0.mlp.experts.gate_up_proj", gu, arch, r, R),
                           shard_tensor("model.layers.0.mlp.experts.down_proj", down, arch, r, R), e) for r in range(R))
        torch.testing.assert_close(parts, expert(gu, down, e), atol=1e-3, rtol=1e-4)
    # replicated tensors pass through, biases of row-split outputs live on rank 0 only
    emb = torch.randn(128, H)
    assert shard_tensor("model.embed_tokens.weight", emb, arch, 1, R) is emb
    b = torch.randn(H)
    assert shard_tensor("model.layers.0.mlp.down_proj.bias", b, arch, 1, R).abs().sum() == 0
    assert shard_tensor("model.layers.0.mlp.down_proj.bias", b, arch, 0, R) is b


def test_tensor_parallel_engine_in_lockstep_matches_the_single_engine():
    """Two gloo ranks: sharded weights, per-layer sums, rank 0 announcing requests and broadcasting its
    samples; the greedy tokens must be those of the unsharded engine."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(root))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29617", "-m", "tests.distributed.tp_engine",
                        "--batch", "5", "--prompt", "24", "--tokens", "8"], env=env, capture_output=True, text=True,
                       timeout=600, cwd=str(root))
    assert r.returncode == 0 and "TP_SELFTEST_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert "identical_sequences=5/5" in r.stdout


def test_expert_parallel_engine_matches_the_single_engine(free_port):
    """Two gloo ranks, experts split by index (``enable_expert_parallel``): every rank routes all tokens, runs the
    pairs of the experts it owns, and the layer's reduction sums the partial outputs."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(root))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(free_port), "-m",
                        "tests.distributed.tp_engine", "--batch", "5", "--prompt", "24", "--tokens", "8",
                        "--expert-parallel"], env=env, capture_output=True, text=True, timeout=600, cwd=str(root))
    assert r.returncode == 0 and "TP_SELFTEST_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert "identical_sequences=5/5" in r.stdout


def test_range_plan_drops_the_pairs_of_other_ranks():
    from prime_rl_b200.ops import moe as M

    torch.manual_seed(0)
    T, k, E, H = 37, 2, 8, 16
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    w = torch.rand(T, k)
    x = torch.randn(T, H)
    full = M.build_plan(idx, counts, E)
    y_full = M.combine(M.permute(x, full) * 2.0, w, full, T)       # every "expert" doubles its rows
    parts = []
    for lo, hi in ((0, 3), (3, 8)):
        plan = M.build_plan(idx, counts, E, expert_range=(lo, hi))
        assert plan.num_experts == hi - lo and int(plan.total_rows) == int(((counts[lo:hi] + 127) // 128 * 128).sum())
        own = (idx >= lo) & (idx < hi)
        assert torch.equal(plan.slot >= 0, own)
        be = plan.block_expert[plan.block_expert >= 0]
        assert be.numel() == 0 or (int(be.min()) >= 0 and int(be.max()) < hi - lo)
        parts.append(M.combine(M.permute(x, plan) * 2.0, w, plan, T))
    torch.testing.assert_close(parts[0] + parts[1], y_full)


def test_tensor_parallel_http_server_serves_the_same_tokens(tmp_path):
    """The inference entry point with ``tensor_parallel_size = 2`` (two CPU processes under torchrun):
    rank 0 answers HTTP, the other rank follows; greedy tokens equal those of a local unsharded engine."""
    import os
    import signal
    import subprocess
    import sys
    import time
    from pathlib import Path

    import httpx

    from prime_rl_b200.engine.engine import Engine as LocalEngine

    root = Path(__file__).resolve().parents[1]
    port = 18431
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(root))
    log = open(tmp_path / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "prime_rl_b200.entrypoints.inference", "@",
                             str(root / "examples" / "inference.toml"), "--vllm.tensor-parallel-size", "2",
                             "--server.port", str(port), "--server.host", "127.0.0.1", "--vllm.num-pages", "256",
                             "--vllm.data-parallel-rpc-port", "29641"], env=env, cwd=str(root), stdout=log,
                            stderr=subprocess.STDOUT, start_new_session=True)
    try:
        base = f"http://127.0.0.1:{port}"
        deadline = time.time() + 240
        while True:
            try:
                if httpx.get(base + "/health", timeout=2).status_code == 200:
                    break
            except httpx.HTTPError:
                pass
            assert proc.poll() is None and time.time() < deadline, (tmp_path / "server.log").read_text()[-3000:]
            time.sleep(1.0)
        prompt = [5, 17, 99, 3, 42, 8, 250, 77]
        body = {"token_ids": prompt, "sampling_params": {"max_tokens": 6, "temperature": 0.0}}
        r = httpx.post(base + "/inference/v1/generate", json=body, timeout=120)
        assert r.status_code == 200, r.text
        served = r.json()["choices"][0]["token_ids"]
        arch = resolve_arch("tiny-qwen3-moe")
        local = LocalEngine(build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=0), num_pages=64)
        want = local.generate_sync([prompt], SamplingParams(max_tokens=6, temperature=0.0))[0].output
        assert served == want
        assert httpx.post(base + "/pause", timeout=60).status_code == 200
        assert httpx.post(base + "/resume", timeout=60).status_code == 200
        r = httpx.post(base + "/inference/v1/generate", json=body, timeout=120)
        assert r.json()["choices"][0]["token_ids"] == want
        # a weight update from a checkpoint directory: every rank loads its own slices of the new weights
        from prime_rl_b200.trainer.weights import save_hf_checkpoint

        other = build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=7)
        save_hf_checkpoint(other, tmp_path / "step_1", dtype=torch.float32)
        r = httpx.post(base + "/update_weights", json={"weight_dir": str(tmp_path / "step_1")}, timeout=120)
        assert r.status_code == 200 and r.json()["policy_version"] == 1, r.text
        want2 = LocalEngine(other, num_pages=64).generate_sync([prompt], SamplingParams(max_tokens=6, temperature=0.0))[0].output
        r = httpx.post(base + "/inference/v1/generate", json=body, timeout=120)
        assert r.json()["choices"][0]["token_ids"] == want2 and want2 != want
    finally:
        os.killpg(proc.pid, signal.SIGTERM)            # the process group this test started, nothing else
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()


def test_rope_to_cache_fallback_writes_the_same_cache_rows():
    """Without the fused kernel (CPU), ``qkv_rope_to_cache`` is ``qkv_norm_rope`` plus index writes into the pages."""
    from prime_rl_b200 import ops

    torch.manual_seed(0)
    T, nq, nkv, D, pages, ps = 9, 4, 2, 16, 3, 4
    qkv = torch.randn(T, (nq + 2 * nkv) * D)
    qw, kw = torch.rand(D) + 0.5, torch.rand(D) + 0.5
    pos = torch.arange(T, dtype=torch.int32)
    inv_f = ops.inv_freq(D, 1e4)
    slots = torch.randperm(pages * ps)[:T]
    kc, vc = torch.zeros(pages, ps, nkv, D), torch.zeros(pages, ps, nkv, D)
    q, k, v = ops.qkv_rope_to_cache(qkv, qw, kw, pos, inv_f, 1e-6, nq, nkv, D, kc, vc, slots)
    q0, k0, v0 = ops.qkv_norm_rope(qkv, qw, kw, pos, inv_f, 1e-6, nq, nkv, D)
    assert torch.equal(q, q0) and torch.equal(k, k0) and torch.equal(v, v0)
    assert torch.equal(kc.view(-1, nkv, D)[slots], k0) and torch.equal(vc.view(-1, nkv, D)[slots], v0)
    assert int((kc.view(-1, nkv * D).abs().sum(-1) > 0).sum()) == T


def test_small_route_plan_is_gpu_only():
    from prime_rl_b200.ops import moe as moe_ops

    with torch.no_grad():
        assert moe_ops.route_and_plan_small(torch.randn(4, 8), 2) is None


def test_cached_prefix_pages_count_as_available_and_are_evicted_on_demand():
    """Pages that only the prefix cache still holds must not block admission: they are counted as available
    and reclaimed when the free list runs dry."""
    from prime_rl_b200.engine.kv_cache import BlockManager, OutOfPages

    bm = BlockManager(num_pages=8, page_size=4)
    toks = list(range(16))
    pages = [bm.alloc() for _ in range(4)]
    bm.register_prefix("s", toks, pages)
    assert bm.num_available == 4 and bm.evictable == 0          # the sequence still holds its pages
    bm.release(pages)
    assert bm.num_free == 4 and bm.evictable == 4 and bm.num_available == 8 and bm.usage == 0.0
    hit = bm.lookup_prefix("s", toks[:8])                       # a new sequence takes two cached pages
    assert hit == pages[:2] and bm.evictable == 2 and bm.num_available == 6
    got = [bm.alloc() for _ in range(6)]                        # 4 free + 2 reclaimed from the cache
    assert len(set(got)) == 6 and not set(got) & set(hit)
    assert bm.num_available == 0
    import pytest

    with pytest.raises(OutOfPages):
        bm.alloc()
    bm.release(hit)
    assert bm.evictable == 2                                    # back to cache-only
    bm.clear_prefix_cache()
    assert bm.evictable == 0 and bm.num_free == 2


def test_preempted_requests_keep_their_kv_in_host_memory_and_resume_without_a_second_prefill():
    """Too few pages for all requests at once: the engine preempts. With a host budget the victim's K / V is
    swapped out and back in (same tokens as an engine with plenty of pages, no extra prompt tokens processed);
    without one, or past the budget, it is recomputed."""
    arch = resolve_arch("tiny-qwen3")
    model = build_model(arch, device="cpu", dtype=torch.float32)
    torch.manual_seed(0)
    prompts = [torch.randint(0, arch.vocab_size, (40,)).tolist() for _ in range(6)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    roomy = Engine(model, num_pages=256, page_size=16, enable_prefix_cache=False)
    want = [r.output for r in roomy.generate_sync(prompts, sp)]
    assert roomy.stats["preemptions"] == 0

    tight = Engine(model, num_pages=24, page_size=16, enable_prefix_cache=False, kv_offload_bytes=1 << 30)
    got = tight.generate_sync(prompts, sp)
    assert [r.output for r in got] == want
    assert tight.stats["preemptions"] > 0 and tight.stats["kv_swap_outs"] == tight.stats["kv_swap_ins"] > 0
    assert tight.stats["prompt_tokens"] == roomy.stats["prompt_tokens"]        # nothing was prefilled twice
    assert tight.kv_offloaded == 0 and tight.cache.blocks.num_free == 24

    plain = Engine(model, num_pages=24, page_size=16, enable_prefix_cache=False)
    again = plain.generate_sync(prompts, sp)
    assert [r.output for r in again] == want and plain.stats["preemptions"] > 0
    assert plain.stats.get("kv_swap_outs", 0) == 0
    assert plain.stats["prompt_tokens"] > roomy.stats["prompt_tokens"]          # recomputed on re-admission

    small = Engine(model, num_pages=24, page_size=16, enable_prefix_cache=False, kv_offload_bytes=1)
    assert [r.output for r in small.generate_sync(prompts, sp)] == want          # budget too small: falls back
    assert small.stats.get("kv_swap_outs", 0) == 0


@pytest.mark.parametrize("name", ["tiny-nemotron-h", "tiny-qwen3.5-moe", "tiny-glm-moe-dsa", "tiny-deepseek-v4"])
def test_engine_serves_the_recurrent_state_families(name):
    """(GLM-MoE-DSA: multi-head latent attention over the keys a sparse indexer selects; the engine keeps the latent K / V
    row and the indexer key of every token per sequence and layer. DeepSeek-V4: shared K / V rows, compressed entries
    formed as their source tokens arrive, a lightning indexer over the entries, hyper-connection streams.) Mamba-2 / gated delta-net layers next to attention: the engine keeps a convolution tail and a recurrent state per
    sequence and layer, prefills in chunks from the stored state and decodes with one batched recurrence step. Greedy
    tokens and their log-probabilities must be those of the model's own forward over the whole sequence."""
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.engine.hybrid import HybridRunner
    from prime_rl_b200.engine.sampler import SamplingParams
    from prime_rl_b200.models import SeqInfo, build_model, resolve_arch

    arch = resolve_arch(name)
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=0).eval()
    eng = Engine(model, num_pages=256, page_size=16, max_model_len=256, max_prefill_tokens=48)
    assert isinstance(eng.runner, HybridRunner) and not eng.enable_prefix_cache
    g = torch.Generator().manual_seed(1)
    # 100 tokens: longer than one prefill step, so the scans continue from a stored state; the short prompts share steps
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (20, 100, 7, 33)]
    out = eng.generate_sync(prompts, SamplingParams(max_tokens=9, temperature=0.0))
    for p, r in zip(prompts, out):
        assert len(r.output) == 9
        ids = torch.tensor(p + r.output)
        with torch.no_grad():
            h = model(ids, SeqInfo.from_lengths([len(ids)], torch.device("cpu")))
            lp = torch.log_softmax(h.float() @ model.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            t = len(p) - 1 + i
            assert int(lp[t].argmax()) == tok
            assert abs(float(lp[t, tok]) - r.logprobs[i]) < 1e-3
    # the states went away with the requests
    assert all(not r.kv.pages for r in out)


@pytest.mark.parametrize("name", ["tiny-nemotron-h", "tiny-qwen3.5-moe", "tiny-qwen3-moe"])
def test_weight_broadcast_groups_follow_the_checkpoint_naming_of_every_family(name):
    """The in-memory weight broadcast announces a number of layer groups and then sends them; the groups are formed
    from checkpoint-layout names, whose layer prefix differs between families (``model.layers``, ``backbone.layers``)."""
    from prime_rl_b200.models import convert
    from prime_rl_b200.transports.weights.nccl import layer_groups

    arch = resolve_arch(name)
    model = build_model(arch, device="cpu", dtype=torch.float32)
    hf = layer_groups(list(convert.model_state(model, "hf")))
    native = layer_groups(list(convert.model_state(model, "native")))
    assert len(hf) == len(native) == arch.num_hidden_layers + 1


def test_prefill_decode_disaggregation_through_the_router(tmp_path):
    """One prefill engine and one decode engine behind the router: the prompt runs on the first, its K / V travel as
    a file, the second continues without a prefill step; tokens and log-probabilities are those of a single engine.
    Admin calls reach both roles."""
    import asyncio

    import httpx

    from prime_rl_b200.engine.router import Router, build_app as build_router
    from prime_rl_b200.engine.server import build_app

    arch = resolve_arch("tiny-qwen3")
    mk = lambda: Engine(build_model(arch, device="cpu", dtype=torch.float32, seed=3), num_pages=128)
    single = mk()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (20, 37, 5)]
    want = single.generate_sync(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    pre, dec = mk().start(), mk().start()
    router = Router(["http://decode"], transports=[httpx.ASGITransport(app=build_app(dec, "tiny-qwen3"))],
                    prefill_urls=["http://prefill"],
                    prefill_transports=[httpx.ASGITransport(app=build_app(pre, "tiny-qwen3"))])
    app = build_router(router)

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://router") as c:
            for p, w in zip(prompts, want):
                body = {"token_ids": p, "sampling_params": {"max_tokens": 6, "temperature": 0.0},
                        "kv_transfer_dir": str(tmp_path)}
                r = await c.post("/inference/v1/generate", json=body)
                assert r.status_code == 200, r.text
                ch = r.json()["choices"][0]
                assert ch["token_ids"] == w.output and ch["finish_reason"] == "length"
                assert max(abs(a - b) for a, b in zip(ch["logprobs"], w.logprobs)) < 1e-4
            # several samples of one prompt: one hand-off each
            r = await c.post("/inference/v1/generate", json={"token_ids": prompts[0], "kv_transfer_dir": str(tmp_path),
                                                            "sampling_params": {"max_tokens": 4, "temperature": 1.0, "n": 3}})
            assert r.status_code == 200 and [c_["index"] for c_ in r.json()["choices"]] == [0, 1, 2]
            assert r.json()["usage"]["completion_tokens"] == 12
            # a request that ends at its first token never reaches the decode engine
            r = await c.post("/inference/v1/generate", json={"token_ids": prompts[1], "kv_transfer_dir": str(tmp_path),
                                                            "sampling_params": {"max_tokens": 1, "temperature": 0.0}})
            assert r.status_code == 200 and r.json()["choices"][0]["token_ids"] == want[1].output[:1]
            assert (await c.post("/pause")).json()["replicas"] == 2 and pre.paused and dec.paused
            assert (await c.post("/resume")).status_code == 200

    try:
        asyncio.run(go())
    finally:
        pre.shutdown()
        dec.shutdown()
    assert router.handoffs == 6
    assert dec.stats["prompt_tokens"] == 0 and dec.stats["kv_imports"] == 6          # the decode engine never prefilled
    assert pre.stats["generation_tokens"] == 7                                       # one token per prompt run
    assert not list(tmp_path.glob("prb_kv_*"))                                       # every K / V file was consumed
    assert pre.cache.blocks.num_available == 128 and dec.cache.blocks.num_available == 128


@pytest.mark.slow
def test_disaggregated_deployment_as_processes(tmp_path, free_port):
    """``deployment.type = "disaggregated"`` on one node: one prefill and one decode engine process and the router in
    front; greedy tokens equal those of a local engine, and the decode engine reports no prompt tokens."""
    import os
    import signal
    import subprocess
    import sys
    import time
    from pathlib import Path

    import httpx

    root = Path(__file__).resolve().parents[1]
    port = free_port
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(root))
    log = open(tmp_path / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "prime_rl_b200.entrypoints.inference", "@",
                             str(root / "examples" / "inference.toml"), "--deployment.type", "disaggregated",
                             "--deployment.num-prefill-replicas", "1", "--deployment.num-decode-replicas", "1",
                             "--server.port", str(port), "--server.host", "127.0.0.1", "--vllm.num-pages", "256"],
                            env=env, cwd=str(root), stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    try:
        base = f"http://127.0.0.1:{port}"
        deadline = time.time() + 240
        while True:
            try:
                if httpx.get(base + "/health", timeout=2).status_code == 200:
                    break
            except httpx.HTTPError:
                pass
            assert proc.poll() is None and time.time() < deadline, (tmp_path / "server.log").read_text()[-3000:]
            time.sleep(1.0)
        prompt = [5, 17, 99, 3, 42, 8, 250, 77, 12, 900, 31]
        body = {"token_ids": prompt, "sampling_params": {"max_tokens": 6, "temperature": 0.0}}
        r = httpx.post(base + "/inference/v1/generate", json=body, timeout=120)
        assert r.status_code == 200, r.text
        arch = resolve_arch("tiny-qwen3-moe")
        local = Engine(build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=0), num_pages=64)
        want = local.generate_sync([prompt], SamplingParams(max_tokens=6, temperature=0.0))[0].output
        assert r.json()["choices"][0]["token_ids"] == want
        st = httpx.get(base + "/router/state", timeout=10).json()
        assert st["handoffs"] == 1 and len(st["prefill_urls"]) == 1
        decode_metrics = httpx.get(f"http://127.0.0.1:{port + 1}/metrics", timeout=10).text
        assert "vllm:prompt_tokens_total 0" in decode_metrics
    finally:
        os.killpg(proc.pid, signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()


def test_engine_serves_image_inputs_like_the_multimodal_forward():
    """A prompt with two images: the engine runs the vision tower once, puts the features in place of the placeholder
    embeddings, rotates with three-axis positions (generated tokens continue after the largest image position), and
    must give the tokens and log-probabilities of the multimodal model's own forward over the finished sequence. A
    text-only request in the same batch is unaffected."""
    from prime_rl_b200.engine.engine import Request
    from prime_rl_b200.models import vision

    torch.manual_seed(12)
    vc = vision.VisionConfig(depth=2, hidden_size=32, intermediate_size=64, num_heads=4, patch_size=4,
                             temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=64)
    arch = resolve_arch("tiny-qwen3.5-moe")
    lm = build_model(arch, device="cpu", dtype=torch.float32, seed=3).eval()
    image_token = arch.vocab_size - 1
    mm = vision.MultimodalLM(lm, vc, image_token, mrope_section=(2, 1, 1), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])
    pixels = torch.randn(4 * 6 + 2 * 2, 3 * 2 * 4 * 4)
    prompt = torch.randint(0, arch.vocab_size - 1, (20,))
    prompt[3:9] = image_token
    prompt[15:16] = image_token
    text = torch.randint(0, arch.vocab_size - 1, (11,)).tolist()
    eng = Engine(lm, num_pages=128, max_model_len=128, max_prefill_tokens=16, vision=mm.visual,
                 image_token_id=image_token, mrope_section=(2, 1, 1))
    params = SamplingParams(max_tokens=6, temperature=0.0)
    reqs = [eng.submit(Request(prompt=prompt.tolist(), params=params,
                               mm={"pixel_values": pixels, "image_grid_thw": grid})),
            eng.submit(Request(prompt=text, params=params))]
    while any(r.finish_reason is None for r in reqs):
        eng.step()
    for r, images in zip(reqs, (True, False)):
        ids = torch.tensor(r.prompt + r.output)
        seq = SeqInfo.from_lengths([len(ids)], "cpu")
        with torch.no_grad():
            h = mm(ids, seq, pixels, grid) if images else lm(ids, seq)
            lp = torch.log_softmax(h.float() @ lm.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            t = len(r.prompt) - 1 + i
            assert int(lp[t].argmax()) == tok
            assert abs(float(lp[t, tok]) - r.logprobs[i]) < 1e-3


def test_image_inputs_travel_from_the_client_to_the_engine_and_into_the_sample():
    """Orchestrator client -> HTTP server -> engine with a vision tower, and the same images into the training sample."""
    import asyncio
    from types import SimpleNamespace

    import httpx
    import numpy as np

    from prime_rl_b200.engine.server import build_app
    from prime_rl_b200.models import vision
    from prime_rl_b200.orchestrator.algo import Algorithm
    from prime_rl_b200.orchestrator.clients import InferenceClient
    from prime_rl_b200.orchestrator.types import Rollout, Turn

    torch.manual_seed(12)
    vc = vision.VisionConfig(depth=1, hidden_size=32, intermediate_size=64, num_heads=4, patch_size=4,
                             temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=64)
    arch = resolve_arch("tiny-qwen3.5-moe")
    lm = build_model(arch, device="cpu", dtype=torch.float32, seed=3).eval()
    image_token = arch.vocab_size - 1
    tower = vision.VisionTower(vc, dtype=torch.float32).eval()
    grid = [[1, 4, 4]]
    pixels = torch.randn(16, 3 * 2 * 4 * 4)
    prompt = torch.randint(0, arch.vocab_size - 1, (12,))
    prompt[2:6] = image_token
    mm = {"pixel_values": pixels.numpy(), "image_grid_thw": grid, "image_token_id": image_token}
    local = Engine(lm, num_pages=64, max_model_len=64, vision=tower, image_token_id=image_token, mrope_section=(2, 1, 1))
    from prime_rl_b200.engine.engine import Request

    want = local.submit(Request(prompt=prompt.tolist(), params=SamplingParams(max_tokens=5, temperature=0.0),
                                mm={"pixel_values": pixels, "image_grid_thw": torch.tensor(grid)}))
    while want.finish_reason is None:
        local.step()
    eng = Engine(lm, num_pages=64, max_model_len=64, vision=tower, image_token_id=image_token,
                 mrope_section=(2, 1, 1)).start()
    app = build_app(eng, "tiny")

    async def go():
        cfg = SimpleNamespace(base_url="http://engine/v1", api_key_var="NONE", timeout=60, headers={}, name="tiny")
        http = httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://engine")
        body = {"token_ids": prompt.tolist(), "sampling_params": {"max_tokens": 5, "temperature": 0.0}}
        import base64

        px = np.ascontiguousarray(pixels.numpy())
        body["multi_modal_data"] = {"pixel_values": {"dtype": "float32", "shape": list(px.shape),
                                                     "data": base64.b64encode(px.tobytes()).decode()},
                                    "image_grid_thw": grid}
        r = await http.post("/inference/v1/generate", json=body)
        assert r.status_code == 200, r.text
        await http.aclose()
        return r.json()["choices"][0]

    try:
        ch = asyncio.run(go())
    finally:
        eng.shutdown()
    assert ch["token_ids"] == want.output
    turn = Turn(prompt.tolist(), ch["token_ids"], ch["logprobs"], mm=mm)
    ro = Rollout(env_name="e", task_id=0, group_id="g", turns=[turn], reward=1.0, policy_version=0)
    ro.advantage = 0.5
    (sample,) = Algorithm(None).to_samples(ro)
    assert sample.mm_kwargs["pixel_values"].shape == [16, 96] and sample.mm_kwargs["image_grid_thw"].shape == [1, 3]
    assert sample.mm_token_type_ids[2:6] == [1, 1, 1, 1] and sum(sample.mm_token_type_ids) == 4


@pytest.mark.parametrize("name", ["tiny-nemotron-h", "tiny-deepseek-v4"])
def test_samples_of_one_prompt_fork_the_prefill_in_the_recurrent_state_runner(name):
    """A group of samples of one prompt (what the RL orchestrator sends): the prompt runs once, the other samples take
    copy-on-write pages and copies of the recurrent / latent state; every sample must still be scored as by the
    model's own forward, and greedy samples must coincide."""
    from prime_rl_b200.engine.engine import Request

    arch = resolve_arch(name)
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=0).eval()
    eng = Engine(model, num_pages=256, page_size=16, max_model_len=256)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, arch.vocab_size, (27,), generator=g).tolist()
    other = torch.randint(0, arch.vocab_size, (9,), generator=g).tolist()
    sampled = [eng.submit(Request(prompt=prompt, params=SamplingParams(max_tokens=7, temperature=1.0, seed=10 + i)))
               for i in range(4)]
    greedy = [eng.submit(Request(prompt=p, params=SamplingParams(max_tokens=7, temperature=0.0)))
              for p in (prompt, other, prompt)]
    reqs = sampled + greedy
    while any(r.finish_reason is None for r in reqs):
        eng.step()
    assert eng.stats["prefill_forks"] == 5                      # six requests share the long prompt: one ran it
    assert eng.stats["prompt_tokens"] == len(prompt) + len(other)
    assert greedy[0].output == greedy[2].output
    assert len({tuple(r.output) for r in sampled}) > 1          # the samples are independent draws
    for r in reqs:
        ids = torch.tensor(r.prompt + r.output)
        with torch.no_grad():
            h = model(ids, SeqInfo.from_lengths([len(ids)], torch.device("cpu")))
            lp = torch.log_softmax(h.float() @ model.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            assert abs(float(lp[len(r.prompt) - 1 + i, tok]) - r.logprobs[i]) < 1e-3
    assert eng.cache.blocks.num_available == 256


def test_preemption_in_the_recurrent_state_runner_restarts_from_the_tokens():
    """Too few pages for all requests: the preempted ones lose pages and state and later run prompt + output so far
    again; their final tokens and log-probabilities are still those of the model's own forward."""
    from prime_rl_b200.engine.engine import Request

    arch = resolve_arch("tiny-nemotron-h")
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=0).eval()
    eng = Engine(model, num_pages=9, page_size=16, max_model_len=128)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (30, 28, 31)]
    reqs = [eng.submit(Request(prompt=p, params=SamplingParams(max_tokens=24, temperature=0.0))) for p in prompts]
    while any(r.finish_reason is None for r in reqs):
        eng.step()
    assert eng.stats["preemptions"] > 0
    for r in reqs:
        assert len(r.output) == 24
        ids = torch.tensor(r.prompt + r.output)
        with torch.no_grad():
            h = model(ids, SeqInfo.from_lengths([len(ids)], torch.device("cpu")))
            lp = torch.log_softmax(h.float() @ model.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            t = len(r.prompt) - 1 + i
            assert int(lp[t].argmax()) == tok and abs(float(lp[t, tok]) - r.logprobs[i]) < 1e-3
    assert eng.cache.blocks.num_available == 9


def test_a_group_of_samples_is_admitted_as_one_prompt_in_the_recurrent_state_runner():
    """Eight samples of a prompt longer than an eighth of the prefill budget: they are admitted together (the copies
    cost no prompt tokens) and the prompt runs once."""
    from prime_rl_b200.engine.engine import Request

    arch = resolve_arch("tiny-qwen3.5-moe")
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=0).eval()
    eng = Engine(model, num_pages=256, page_size=16, max_model_len=256, max_prefill_tokens=64)
    prompt = torch.randint(0, arch.vocab_size, (40,), generator=torch.Generator().manual_seed(6)).tolist()
    reqs = [eng.submit(Request(prompt=prompt, params=SamplingParams(max_tokens=3, temperature=1.0, seed=i))) for i in range(8)]
    eng.step()
    assert eng.stats["prompt_tokens"] == 40 and eng.stats["prefill_forks"] == 7
    while any(r.finish_reason is None for r in reqs):
        eng.step()
    assert eng.stats["prompt_tokens"] == 40 and all(len(r.output) == 3 for r in reqs)
