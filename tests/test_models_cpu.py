import torch

from prime_rl_b200.models import SeqInfo, apply_lora, build_model, convert, resolve_arch
from prime_rl_b200.models.config import ModelArch
from prime_rl_b200.ops import attention as A
from prime_rl_b200.ops import lm_head, moe


def _tiny(name="tiny-qwen3-moe", **over):
    arch = resolve_arch(name, over or None)
    return arch, build_model(arch, device="cpu", dtype=torch.float32)


def test_packed_documents_do_not_interact():
    arch, m = _tiny("tiny-qwen3")
    ids = torch.randint(0, arch.vocab_size, (96,))
    packed = m(ids, SeqInfo.from_lengths([40, 56], "cpu"))
    a = m(ids[:40], SeqInfo.from_lengths([40], "cpu"))
    b = m(ids[40:], SeqInfo.from_lengths([56], "cpu"))
    assert torch.allclose(packed[:40], a, atol=1e-4) and torch.allclose(packed[40:], b, atol=1e-4)


def test_fused_head_matches_full_logits():
    arch, m = _tiny("tiny-qwen3")
    T = 50
    h = torch.randn(T, arch.hidden_size, requires_grad=True)
    labels = torch.randint(0, arch.vocab_size, (T,))
    it = 0.5 + torch.rand(T)
    lp, ent = lm_head.logprob_entropy_ref(h, m.output_weight, labels, it, chunk=16)
    z = (h @ m.output_weight.t()) * it[:, None]
    want = torch.log_softmax(z, -1).gather(1, labels[:, None]).squeeze(1)
    p = torch.softmax(z, -1)
    assert torch.allclose(lp, want, atol=1e-5)
    assert torch.allclose(ent, -(p * torch.log_softmax(z, -1)).sum(-1), atol=1e-4)


def test_moe_matches_dense_loop():
    arch, m = _tiny()
    layer = m.model.layers[0].mlp
    x = torch.randn(70, arch.hidden_size)
    y = layer(x, SeqInfo.from_lengths([70], "cpu"))
    idx, w, _, _ = layer.router(x)
    I = arch.moe_intermediate_size
    want = torch.zeros_like(x)
    for t in range(70):
        for j in range(arch.num_experts_per_tok):
            e = int(idx[t, j])
            gu = layer.experts.gate_up_proj[e] @ x[t]
            hmid = torch.nn.functional.silu(gu[:I]) * gu[I:]
            want[t] += w[t, j] * (layer.experts.down_proj[e] @ hmid)
    assert torch.allclose(y, want, atol=1e-4)


def test_plan_is_128_aligned_and_complete():
    idx = torch.randint(0, 8, (300, 2), dtype=torch.int32)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=8).to(torch.int32)
    plan = moe.build_plan(idx, counts, 8)
    offs = plan.expert_offset.long()
    assert (offs % 128 == 0).all()
    slot = plan.slot.long()
    assert ((slot >= offs[idx.long()]) & (slot < offs[idx.long() + 1])).all()
    assert slot.unique().numel() == slot.numel()
    assert (plan.row_src[slot.reshape(-1)].long() == torch.arange(600)).all()


def test_layout_round_trips_and_hf_names():
    arch, m = _tiny()
    prime = convert.model_state(m, "prime")
    assert "model.layers.0.self_attn.q_proj.weight" in prime
    assert prime["model.layers.0.mlp.experts.gate_proj"].shape == (8, arch.moe_intermediate_size, arch.hidden_size)
    assert "model.layers.0.mlp.router.gate.weight" in prime
    hf = convert.model_state(m, "hf")
    assert "model.layers.1.mlp.experts.7.down_proj.weight" in hf and "model.layers.0.mlp.gate.weight" in hf
    back = convert.hf_to_native({k: v.clone() for k, v in hf.items()}, arch)
    for k, v in m.state_dict().items():
        if not k.endswith("inv_freq"):
            assert torch.equal(back[k], v), k


def test_lora_freezes_base_and_starts_as_identity():
    arch, m = _tiny()
    ids = torch.randint(0, arch.vocab_size, (64,))
    seq = SeqInfo.from_lengths([64], "cpu")
    before = m(ids, seq)
    apply_lora(m, 4, 8.0, ["q_proj", "k_proj", "v_proj", "o_proj", "experts"])
    after = m(ids, seq)
    assert torch.allclose(before, after, atol=1e-6)  # B = 0 at init
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    after.sum().backward()
    assert all(p.grad is not None for n, p in m.named_parameters() if p.requires_grad)
    peft = convert.lora_to_peft(m)
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in peft
    assert "base_model.model.model.layers.0.mlp.experts.gate_proj.lora_B.weight" in peft


def test_attention_reference_window_and_sinks():
    T, H, D = 24, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, H, D), torch.randn(T, H, D)
    cu = torch.tensor([0, 10, 24], dtype=torch.int32)
    full = A.attention_ref(q, k, v, cu)
    win = A.attention_ref(q, k, v, cu, window=1)
    assert torch.allclose(win, v, atol=1e-5)  # window of 1 attends to itself only
    sink = A.attention_ref(q, k, v, cu, sinks=torch.full((H,), 50.0))
    assert sink.abs().max() < 1e-3 * full.abs().max() + 1e-3  # a huge sink takes all the mass


def test_hf_config_interchange():
    arch = resolve_arch("qwen3-30b-a3b")
    assert arch.param_count() > 30e9 and arch.param_count(active_only=True) < 3.5e9
    again = ModelArch.from_hf_config(arch.to_hf_config())
    assert again.num_experts == 128 and again.moe_intermediate_size == 768 and again.qk_norm


def test_laguna_family_gating_per_layer_heads_and_round_trip(tmp_path):
    """Attention output gate, per-layer head counts, dense / sparse layer list, shared expert of
    its own width; HF config and checkpoint names round-trip."""
    import torch

    from prime_rl_b200.models import ModelArch, build_model, convert, resolve_arch
    from prime_rl_b200.models.layers import MoE, SeqInfo

    arch = resolve_arch("tiny-laguna")
    model = build_model(arch, device="cpu", dtype=torch.float32, seed=0)
    layers = model.model.layers
    assert [l.self_attn.nq for l in layers] == [4, 2, 4]
    assert [isinstance(l.mlp, MoE) for l in layers] == [False, True, True]
    assert layers[1].self_attn.g_proj.weight.shape == (2, arch.hidden_size)
    assert layers[1].mlp.shared_experts.down_proj.weight.shape[1] == 96
    assert [l.self_attn.window for l in layers] == [16, None, 16]
    ids = torch.randint(0, arch.vocab_size, (40,))
    seq = SeqInfo(torch.tensor([0, 25, 40], dtype=torch.int32), 25, torch.cat([torch.arange(25), torch.arange(15)]).int())
    h = model(ids, seq)
    assert h.shape == (40, arch.hidden_size) and torch.isfinite(h).all()
    h.sum().backward()
    assert layers[1].self_attn.g_proj.weight.grad.abs().sum() > 0
    # config round trip
    again = ModelArch.from_hf_config(arch.to_hf_config())
    assert again.heads_per_layer == [4, 2, 4] and again.attn_gate == "per_head" and again.shared_width == 96
    assert again.mlp_layer_types == ["dense", "sparse", "sparse"]
    # names: singular shared expert and the bias under `experts`, and back
    hf = convert.model_state(model, "hf")
    assert "model.layers.1.mlp.shared_expert.gate_proj.weight" in hf
    assert "model.layers.1.mlp.experts.e_score_correction_bias" in hf
    assert "model.layers.1.self_attn.g_proj.weight" in hf
    assert hf["model.layers.1.self_attn.q_proj.weight"].shape[0] == 2 * arch.head_dim
    other = build_model(arch, device="cpu", dtype=torch.float32, seed=1)
    convert.load_model_state(other, hf, "hf")
    for (n, a), (_, b) in zip(model.state_dict().items(), other.state_dict().items()):
        assert torch.equal(a, b), n


def test_selective_recomputation_keeps_gemm_outputs_and_matches_full_recomputation():
    """``ac.mode = "selective"``: the re-run of a checkpointed layer replays the kept GEMM outputs instead of
    recomputing them; losses and gradients equal full recomputation and no recomputation at all."""
    from prime_rl_b200.ops import stash

    def grads(keep, ac_every):
        arch, m = _tiny("tiny-qwen3-moe")
        m.train()
        m.ac_every, m.ac_keep = ac_every, keep
        ids = torch.randint(0, arch.vocab_size, (64,), generator=torch.Generator().manual_seed(0))
        seq = SeqInfo.from_lengths([64], "cpu")
        h = m(ids, seq)
        (h.float() ** 2).mean().backward()
        return {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}, seq

    plain, _ = grads(None, None)
    full, seq_full = grads(None, 1)
    sel, seq_sel = grads({"mm", "grouped_mm"}, 1)
    assert seq_full.op_stash is None and seq_sel.op_stash is not None
    st = seq_sel.op_stash.stats
    assert st["recorded"] > 0 and st["replayed"] == st["recorded"] and not seq_sel.op_stash.store
    for n in plain:
        assert torch.allclose(plain[n], full[n], atol=1e-6), n
        assert torch.allclose(plain[n], sel[n], atol=1e-6), n
    assert stash.kinds_from_targets(None) == {"mm", "grouped_mm", "attention"}
    assert stash.kinds_from_targets(["aten::mm", "flash_attn"]) == {"mm", "attention"}
    assert stash.kinds_from_targets([]) == set()


def test_several_lora_adapters_in_one_micro_batch():
    """Tokens are sorted by adapter (``lora_num_tokens``); every token must get its own adapter's update on dense
    projections and on the experts, gradients must stay with the adapter whose tokens produced them, and one
    adapter must reproduce the single-adapter model."""
    from prime_rl_b200.models import SeqInfo, apply_lora, build_model, resolve_arch
    from prime_rl_b200.models.layers import LoRAAdapter, MultiLoRA, set_lora_num_tokens

    torch.manual_seed(0)
    arch = resolve_arch("tiny-qwen3-moe")
    def fresh():
        return build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=1)

    multi = fresh()
    apply_lora(multi, 4, 8.0, ["q_proj", "k_proj", "v_proj", "o_proj", "experts"], num_adapters=2)
    assert any(isinstance(m, MultiLoRA) for m in multi.modules())
    with torch.no_grad():                                    # make the adapters differ and do something
        for i, m in enumerate(mm for mm in multi.modules() if isinstance(mm, LoRAAdapter)):
            for b in m.lora_B:
                b.normal_(0, 0.05 * (1 + i % 2))
    T = 24
    ids = torch.randint(0, arch.vocab_size, (T,))
    seq = SeqInfo.from_lengths([T], torch.device("cpu"))

    def single_from(k):
        m = fresh()
        apply_lora(m, 4, 8.0, ["q_proj", "k_proj", "v_proj", "o_proj", "experts"])
        src = {n: p for n, p in multi.named_parameters() if "lora_" in n}
        with torch.no_grad():
            for n, p in m.named_parameters():
                if "lora_" in n:
                    # layers.N.self_attn.qkv_proj.lora.lora_A  <-  ...qkv_proj.lora.<k>.lora_A
                    head, tail = n.rsplit(".lora_", 1)
                    p.copy_(src[f"{head}.{k}.lora_{tail}"])
        return m

    set_lora_num_tokens(torch.tensor([10, 14], dtype=torch.int32))
    out = multi(ids, seq)
    h = out[0] if isinstance(out, tuple) else out
    set_lora_num_tokens(None)
    ref0 = single_from(0)(ids[:10], SeqInfo.from_lengths([10], torch.device("cpu")))
    ref0 = ref0[0] if isinstance(ref0, tuple) else ref0
    # causal model: the first 10 tokens only see adapter-0 tokens, so they must match the single-adapter model
    assert torch.allclose(h[:10], ref0, atol=2e-4, rtol=1e-3)
    # all tokens on adapter 1 == the single-adapter model built from adapter 1
    set_lora_num_tokens(torch.tensor([0, T], dtype=torch.int32))
    h1 = multi(ids, seq)
    h1 = h1[0] if isinstance(h1, tuple) else h1
    ref1 = single_from(1)(ids, seq)
    ref1 = ref1[0] if isinstance(ref1, tuple) else ref1
    assert torch.allclose(h1, ref1, atol=2e-4, rtol=1e-3)
    # gradients: with every token on adapter 1, adapter 0 gets exactly zero
    h1.float().pow(2).mean().backward()
    set_lora_num_tokens(None)
    g0 = [p.grad for n, p in multi.named_parameters() if ".0.lora_" in n and p.grad is not None]
    g1 = [p.grad for n, p in multi.named_parameters() if ".1.lora_" in n and p.grad is not None]
    assert g1 and all(float(g.abs().sum()) == 0.0 for g in g0) and any(float(g.abs().sum()) > 0 for g in g1)


def test_parameter_sharding_runtime_keeps_the_running_layer_bound_when_the_backward_pass_turns():
    """Two gather buffers, the next layer gathered ahead: at the top of the backward pass (the last layer of the
    forward pass is recomputed first, nothing was gathered ahead of it) the rotation must not hand the buffer of
    the layer that is about to run to the layer gathered ahead. Single process, sharding over one rank."""
    from prime_rl_b200.models import SeqInfo, build_model, resolve_arch
    from prime_rl_b200.parallel.fsdp import install_fsdp

    arch = resolve_arch("tiny-qwen3").model_copy(update={"num_hidden_layers": 5})
    ref = build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=0)
    m = build_model(arch, device=torch.device("cpu"), dtype=torch.float32, seed=0)
    ref.ac_every = m.ac_every = 1
    _, runtime = install_fsdp(m, None, pool=2, prefetch=True)
    ref.train(), m.train()
    ids = torch.randint(0, arch.vocab_size, (64,))
    seq = SeqInfo.from_lengths([64], torch.device("cpu"))

    def loss(model):
        out = model(ids, seq)
        h = out[0] if isinstance(out, tuple) else out
        return h.float().pow(2).mean()

    want = loss(ref)
    want.backward()
    runtime.before_forward()
    got = loss(m)
    got.backward()                               # raised "about to run without its parameters" before the fix
    runtime.finish_backward()
    assert torch.allclose(got, want, atol=1e-6)
    assert runtime.stats["gathers"] == 8         # 5 on the way up, layers 2, 1, 0 again on the way down
