"""Rollout engine on a GPU: paged tensor-core attention, CUDA-graph replay and fp8 weights against
the plain paths of the same engine."""

import pytest
import torch

pytestmark = pytest.mark.gpu

ARCH = dict(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=2, num_attention_heads=8,
            num_key_value_heads=2, head_dim=128, intermediate_size=512, num_experts=8, num_experts_per_tok=2,
            moe_intermediate_size=256, vocab_size=2048)


def _setup(**kw):
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.models import ModelArch, build_model

    dev = torch.device("cuda", 0)
    arch = ModelArch(**ARCH)
    model = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0)
    return arch, model, Engine(model, num_pages=512, page_size=16, enable_prefix_cache=False, max_model_len=256, **kw)


def _greedy(eng, prompts, n=12):
    from prime_rl_b200.engine.sampler import SamplingParams

    return eng.generate_sync(prompts, SamplingParams(max_tokens=n, temperature=0.0))


def test_cuda_graph_decode_matches_eager_decode():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.ops import _runtime as rt

    arch, model, plain = _setup()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (5, 33, 64, 17, 90)]
    ref = _greedy(plain, prompts)
    from prime_rl_b200.engine.engine import Engine

    graphed = Engine(model, num_pages=512, page_size=16, enable_prefix_cache=False, max_model_len=256,
                     use_cuda_graphs=True)
    got = _greedy(graphed, prompts)
    rt.check_status()
    assert graphed.runner._graphs, "no decode graph was captured"
    same = sum(a.output == b.output for a, b in zip(ref, got))
    assert same >= len(prompts) - 1          # bf16 ties may flip one greedy token
    for a, b in zip(ref, got):
        n = min(len(a.logprobs), len(b.logprobs), 4)
        assert all(abs(x - y) < 5e-2 for x, y in zip(a.logprobs[:n], b.logprobs[:n]))


def test_fp8_weight_mode_stays_close_to_bf16():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.engine.runner import StepInput
    from prime_rl_b200.ops import _runtime as rt

    arch, model, eng = _setup()
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, arch.vocab_size, (48,), generator=g).tolist()
    from prime_rl_b200.engine.kv_cache import SequenceKV

    ref, _ = eng.runner.forward([StepInput(SequenceKV(), prompt, want_all_logits=True)])
    from prime_rl_b200.models.model import quantize_fp8_

    assert quantize_fp8_(model) >= 4
    out, _ = eng.runner.forward([StepInput(SequenceKV(), prompt, want_all_logits=True)])
    rt.check_status()
    assert torch.isfinite(out).all()
    rel = (out - ref).norm() / ref.norm()
    assert rel < 0.15, f"fp8 logits deviate by {rel:.3f}"
    agree = (out.argmax(-1) == ref.argmax(-1)).float().mean()
    assert agree > 0.7


def test_sampling_kernel_matches_softmax_statistics_and_logprobs():
    """The one-pass Gumbel-max sampler: greedy rows take the arg-max, sampled rows follow softmax(z / T)
    (checked by frequencies over many draws of a small vocabulary), and the returned log-probability is
    log softmax(z / T) at the drawn token. A seeded generator replays the same tokens."""
    from prime_rl_b200.engine.sampler import sample

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    V, B = 37, 4096
    row = torch.randn(V, device=dev) * 2.0
    logits = row[None, :].repeat(B, 1).contiguous()
    temp = torch.full((B,), 0.7, device=dev)
    temp[:16] = 0.0
    off = torch.zeros(B, dtype=torch.long, device=dev)
    ones = torch.ones(B, device=dev)
    g = torch.Generator(device=dev).manual_seed(11)
    tok, lp, masks = sample(logits, temp, off, ones, generator=g, truncated=False)
    assert masks is None and tok.dtype == torch.long
    assert (tok[:16] == row.argmax()).all()
    ref = torch.log_softmax(row / 0.7, -1)
    torch.testing.assert_close(lp[16:], ref[tok[16:]], atol=2e-4, rtol=0)
    torch.testing.assert_close(lp[:16], torch.log_softmax(row, -1)[tok[:16]], atol=2e-4, rtol=0)
    freq = torch.bincount(tok[16:], minlength=V).float() / (B - 16)
    # standard error of a frequency p over n draws is sqrt(p (1 - p) / n) <= 0.008 here
    assert (freq - ref.exp()).abs().max() < 0.035
    g2 = torch.Generator(device=dev).manual_seed(11)
    tok2, _, _ = sample(logits, temp, off, ones, generator=g2, truncated=False)
    assert torch.equal(tok, tok2)
    tok3, _, _ = sample(logits, temp, off, ones, generator=g2, truncated=False)
    assert not torch.equal(tok, tok3)
    # a large vocabulary with a ragged length and a row pitch wider than V
    wide = torch.randn(8, 151936 + 64, device=dev)
    view = wide[:, :151931]
    t8 = torch.full((8,), 1.3, device=dev)
    tok, lp, _ = sample(view, t8, off[:8], ones[:8], truncated=False)
    torch.testing.assert_close(lp, torch.log_softmax(view / 1.3, -1).gather(1, tok[:, None]).squeeze(1), atol=5e-4, rtol=0)


def test_prefill_on_a_cached_prefix_uses_the_query_slice_kernel_and_matches_a_fresh_prefill():
    """A prompt whose first pages are already cached is prefilled as a query slice [prefix, ctx) against K / V
    gathered from the pages (tensor-core kernel); tokens and log-probabilities must be those of an engine
    that has no prefix cache and prefills the whole prompt."""
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.ops import _runtime as rt

    arch, model, plain = _setup()
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, arch.vocab_size, (80,), generator=g).tolist()
    tails = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (7, 21, 40)]
    prompts = [base + t for t in tails]
    ref = _greedy(plain, prompts, n=6)
    cached = Engine(model, num_pages=512, page_size=16, enable_prefix_cache=True, max_model_len=256)
    _greedy(cached, [base + [1, 2, 3]], n=2)                    # fills the cache with the pages of `base`
    got = _greedy(cached, prompts, n=6)
    rt.check_status()
    assert cached.stats["prefix_hits"] >= 3 * 64               # 80 tokens = 5 pages, at least 4 of them shared
    same = sum(a.output == b.output for a, b in zip(ref, got))
    assert same >= len(prompts) - 1                             # bf16 ties may flip one greedy token
    for a, b in zip(ref, got):
        assert abs(a.logprobs[0] - b.logprobs[0]) < 5e-2


def test_fp8_engine_without_bf16_copies_serves_and_takes_weight_updates(tmp_path):
    """``keep_bf16_weights=False`` releases the bf16 storage of every quantised projection. The engine must
    give the same greedy tokens as the fp8 engine that keeps them, and a weight update from a checkpoint
    directory must be quantised straight into the fp8 copies."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.models import ModelArch, build_model
    from prime_rl_b200.ops import _runtime as rt
    from prime_rl_b200.trainer.weights import save_hf_checkpoint

    dev = torch.device("cuda", 0)
    arch = ModelArch(**ARCH)
    kw = dict(num_pages=512, page_size=16, enable_prefix_cache=False, max_model_len=256, weight_dtype="fp8")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (9, 40, 64)]
    keep = Engine(build_model(arch, device=dev, dtype=torch.bfloat16, seed=0), **kw)
    lean = Engine(build_model(arch, device=dev, dtype=torch.bfloat16, seed=0), keep_bf16_weights=False, **kw)
    layer = lean.model.model.layers[0]
    assert layer.mlp.experts.gate_up_proj.numel() == 0 and layer.self_attn.qkv_proj.weight.numel() == 0
    a, b = _greedy(keep, prompts), _greedy(lean, prompts)
    assert [r.output for r in a] == [r.output for r in b]
    # new weights arrive as an HF directory
    other = build_model(arch, device=dev, dtype=torch.bfloat16, seed=7)
    save_hf_checkpoint(other, tmp_path / "w")
    lean.update_weights_from_dir(str(tmp_path / "w"))
    keep.update_weights_from_dir(str(tmp_path / "w"))
    assert layer.mlp.experts.gate_up_proj.numel() == 0
    a, b = _greedy(keep, prompts), _greedy(lean, prompts)
    rt.check_status()
    assert [r.output for r in a] == [r.output for r in b]
    fresh = Engine(other, **kw)
    c = _greedy(fresh, prompts)
    assert sum(x.output == y.output for x, y in zip(b, c)) >= 2


@pytest.mark.parametrize("weight_dtype,bound", [("bf16", 0.015), ("fp8", 0.015)])
def test_trainer_rescoring_of_engine_rollouts_stays_under_the_mismatch_kl_bar(weight_dtype, bound):
    """The acceptance bar for a model family: sample 256 tokens per prompt with the engine (temperature 1),
    re-score the same tokens with the trainer's forward and fused head, and require the mismatch KL
    ``r - log r - 1`` (``r`` = trainer probability / engine probability of the sampled token) to stay under
    0.015 on average (reference: docs/development.md:140, tests/integration/test_reverse_text.py:116-117)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.engine.sampler import SamplingParams
    from prime_rl_b200.models import ModelArch, SeqInfo, build_model
    from prime_rl_b200.ops import _runtime as rt

    dev = torch.device("cuda", 0)
    arch = ModelArch(**{**ARCH, "num_hidden_layers": 4, "hidden_size": 512, "moe_intermediate_size": 256})
    engine_model = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0)
    trainer_model = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0).eval()
    eng = Engine(engine_model, num_pages=1024, page_size=16, enable_prefix_cache=False, max_model_len=512,
                 weight_dtype=weight_dtype, use_cuda_graphs=True)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (16, 33, 48, 64, 20, 57, 40, 25)]
    reqs = eng.generate_sync(prompts, SamplingParams(max_tokens=256, temperature=1.0))
    rt.check_status()
    kls = []
    with torch.no_grad():
        for r in reqs:
            ids = torch.tensor(r.prompt + r.output, device=dev)
            n_p, n_o = len(r.prompt), len(r.output)
            assert n_o == 256 and len(r.logprobs) == n_o
            hidden = trainer_model(ids, SeqInfo.from_lengths([ids.numel()], dev))
            labels = torch.cat([ids[1:], ids[:1]]).to(torch.int32)
            lp, _ = trainer_model.logprobs_entropy(hidden, labels, None)
            mine = lp[n_p - 1:n_p - 1 + n_o].float()          # position t scores token t + 1
            theirs = torch.tensor(r.logprobs, device=dev)
            log_ratio = mine - theirs
            kls.append((torch.exp(log_ratio) - log_ratio - 1).mean().item())
    rt.check_status()
    mean_kl = sum(kls) / len(kls)
    assert mean_kl < bound, f"mismatch KL {mean_kl:.5f} per sequence {['%.4f' % k for k in kls]}"


def test_samples_of_one_prompt_decode_through_the_shared_prefix_kernel():
    """With the prefix cache on, the samples of a prompt share its pages; the runner groups them and the decode
    step reads the shared pages once per group. Tokens and log-probabilities must be those of an engine without
    prefix sharing (greedy decoding), with and without CUDA graphs."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.ops import _runtime as rt

    arch, model, plain = _setup()
    g = torch.Generator().manual_seed(9)
    base = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (96, 80)]
    tails = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (3, 9, 17, 5, 11, 2)]
    prompts = [base[i % 2] + t for i, t in enumerate(tails)]
    ref = _greedy(plain, prompts, n=20)
    for graphs in (False, True):
        eng = Engine(model, num_pages=512, page_size=16, enable_prefix_cache=True, max_model_len=256,
                     use_cuda_graphs=graphs)
        _greedy(eng, [b + [1, 2] for b in base], n=2)           # fill the cache with the two prompts' pages
        got = _greedy(eng, prompts, n=20)
        rt.check_status()
        st = eng.runner.prefix_stats
        assert st["regroupings"] >= 1 and st["grouped_sequences"] == 6 and st["shared_pages"] >= 4 + 5
        same = sum(a.output == b.output for a, b in zip(ref, got))
        assert same >= len(prompts) - 1
        for a, b in zip(ref, got):
            assert abs(a.logprobs[0] - b.logprobs[0]) < 5e-2


def test_truncated_sampling_kernel_keeps_the_same_set_as_the_sorted_rule():
    """Top-k / top-p without a sort: the kept set must be the prefix of the sorted order that the PyTorch rule
    keeps, samples must fall inside it with the renormalised log-probability, and frequencies must follow it."""
    from prime_rl_b200.engine import sampler as S

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    B, V = 6, 5000
    logits = torch.randn(B, V, device=dev) * 3
    temperature = torch.tensor([1.0, 0.7, 1.0, 1.3, 0.0, 1.0], device=dev)
    top_k = torch.tensor([0, 50, 5, 0, 10, 1], device=dev)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.3, 1.0, 1.0], device=dev)
    # the kept set by the sorted rule
    t = torch.where(temperature <= 0, torch.ones_like(temperature), temperature)
    z = logits / t[:, None]
    srt, idx = torch.sort(z, dim=-1, descending=True)
    probs = torch.softmax(srt, -1)
    keep = (probs.cumsum(-1) - probs) < top_p[:, None]
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V))
    keep &= torch.arange(V, device=dev)[None] < k[:, None]
    want = [set(idx[b][keep[b]].tolist()) for b in range(B)]
    tok, lp, masks = S.sample(logits, temperature, top_k, top_p, want_mask=True)
    for b in range(B):
        got = set(masks[b].tolist())
        assert got == want[b] or (len(want[b]) > S.MAX_MASK and got <= want[b]), (b, len(got), len(want[b]))
        assert int(tok[b]) in want[b]
        kept = torch.tensor(sorted(want[b]), device=dev)
        ref_lp = z[b, tok[b]] - torch.logsumexp(z[b, kept], 0)
        assert abs(float(lp[b]) - float(ref_lp)) < 1e-3
    assert int(tok[4]) == int(logits[4].argmax()) and int(tok[5]) == int(logits[5].argmax())
    # frequencies of row 2 (five kept tokens at most, top-p 0.5)
    kept = sorted(want[2])
    pr = torch.softmax(z[2, torch.tensor(kept, device=dev)], 0)
    counts = torch.zeros(len(kept))
    g = torch.Generator(device=dev).manual_seed(1)
    for _ in range(2000):
        tk, _, _ = S.sample(logits[2:3], temperature[2:3], top_k[2:3], top_p[2:3], generator=g)
        counts[kept.index(int(tk[0]))] += 1
    assert torch.allclose(counts / 2000, pr.cpu(), atol=0.04)


@pytest.mark.parametrize("name", ["tiny-nemotron-h", "tiny-qwen3.5-moe"])
def test_engine_serves_the_recurrent_state_families_on_the_gpu(name):
    """bf16 on the GPU: the engine's incremental path (stored convolution tails and recurrent states, batched one-token
    steps) against the model's own forward over the finished sequences."""
    from prime_rl_b200.engine.engine import Engine
    from prime_rl_b200.engine.hybrid import HybridRunner
    from prime_rl_b200.engine.sampler import SamplingParams
    from prime_rl_b200.models import SeqInfo, build_model, resolve_arch
    from prime_rl_b200.ops import _runtime as rt

    dev = torch.device("cuda", 0)
    arch = resolve_arch(name)
    model = build_model(arch, device=dev, dtype=torch.bfloat16, seed=0).eval()
    eng = Engine(model, num_pages=256, page_size=16, max_model_len=256, max_prefill_tokens=48)
    assert isinstance(eng.runner, HybridRunner)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, arch.vocab_size, (n,), generator=g).tolist() for n in (20, 100, 7, 33)]
    out = eng.generate_sync(prompts, SamplingParams(max_tokens=8, temperature=1.0, seed=3))
    torch.cuda.synchronize()
    rt.check_status()
    worst = 0.0
    for p, r in zip(prompts, out):
        assert len(r.output) == 8
        ids = torch.tensor(p + r.output, device=dev)
        with torch.no_grad():
            h = model(ids, SeqInfo.from_lengths([len(ids)], dev))
            lp = torch.log_softmax(h.float() @ model.output_weight.float().t(), -1)
        for i, tok in enumerate(r.output):
            worst = max(worst, abs(float(lp[len(p) - 1 + i, tok]) - r.logprobs[i]))
    assert worst < 0.08, worst          # bf16 activations, sums in another order between the two paths
