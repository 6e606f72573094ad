"""Logits and gradients of the model stack against HuggingFace ``transformers`` built from the same
configuration (CPU, fp32): the tiny HF model is initialised randomly, its state dict is loaded through
``models/convert.py`` (``layout="hf"``), and both run the same token ids.

Mirrors the reference's per-family parity tests (tests/unit/train/models/test_qwen3_moe.py:61-133 and its
siblings for llama, glm4_moe, gpt_oss): full model, attention-only and MLP-only comparisons through the
hidden states of the first layer, and router replay for the MoE families.
"""

import pytest
import torch

from prime_rl_b200.models import SeqInfo, build_model, convert
from prime_rl_b200.models.config import ModelArch
from prime_rl_b200.trainer.weights import load_hf_checkpoint

transformers = pytest.importorskip("transformers")

T = 48


def _hf_model(cfg):
    torch.manual_seed(0)
    m = transformers.AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").float().eval()
    with torch.no_grad():                 # HF initialises norms to 1 and some biases to 0: make every tensor matter
        for n, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    return m


def _ours(hf, tmp_path):
    """Through a real checkpoint directory: ``save_pretrained`` writes the published layout of the family
    (per-expert tensors for most MoE models) and ``config.json``; this side reads both."""
    d = tmp_path / "hf"
    hf.save_pretrained(d)
    arch = ModelArch.from_pretrained(d)
    m = build_model(arch, device="cpu", dtype=torch.float32)
    load_hf_checkpoint(m, d)
    return arch, m.eval()


def _logits(m, ids):
    h = m(ids, SeqInfo.from_lengths([ids.numel()], "cpu"))
    return h @ m.output_weight.t()


def _compare(hf, ours, arch, atol=2e-4, grads=True):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, arch.vocab_size, (T,), generator=g)
    want = hf(ids[None]).logits[0]
    got = _logits(ours, ids)
    err = (got - want).abs().max().item()
    assert err < atol * max(1.0, want.abs().max().item()), f"logits differ by {err:.3e}"
    if not grads:
        return
    # gradients of a scalar of the logits with respect to the (converted) weights
    w = torch.randn(T, arch.vocab_size, generator=g)
    hf.zero_grad()
    (hf(ids[None]).logits[0] * w).sum().backward()
    for p in ours.parameters():
        p.grad = None
    (_logits(ours, ids) * w).sum().backward()
    # this side's gradients under checkpoint names; transformers keeps expert stacks fused in memory under
    # names that match this side's own ("...mlp.experts.gate_up_proj"), so those are compared natively
    mine = {n: p.grad for n, p in ours.named_parameters() if p.grad is not None}
    mine_hf = convert.native_to_hf(dict(mine), arch)
    checked = 0
    for name, p in hf.named_parameters():
        if p.grad is None:
            continue
        g = mine_hf.get(name)
        if g is None or g.shape != p.grad.shape:
            g = mine.get(name)
        if g is None or g.shape != p.grad.shape:
            continue
        scale = max(1.0, p.grad.abs().max().item())
        assert (g - p.grad).abs().max().item() < 5e-4 * scale, f"gradient of {name} differs"
        checked += 1
    assert checked >= 6, checked


def test_llama_matches_transformers(tmp_path):
    cfg = transformers.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                   rope_theta=10000.0, tie_word_embeddings=False)
    hf = _hf_model(cfg)
    arch, ours = _ours(hf, tmp_path)
    _compare(hf, ours, arch)


def test_qwen2_with_attention_bias_matches_transformers(tmp_path):
    cfg = transformers.Qwen2Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                   tie_word_embeddings=True, use_sliding_window=False)
    hf = _hf_model(cfg)
    arch, ours = _ours(hf, tmp_path)
    assert arch.tie_word_embeddings
    _compare(hf, ours, arch)


def test_qwen3_matches_transformers(tmp_path):
    cfg = transformers.Qwen3Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                   max_position_embeddings=256, tie_word_embeddings=False)
    hf = _hf_model(cfg)
    arch, ours = _ours(hf, tmp_path)
    _compare(hf, ours, arch)


def _qwen3_moe(tmp_path):
    cfg = transformers.Qwen3MoeConfig(vocab_size=320, hidden_size=64, intermediate_size=160, moe_intermediate_size=48,
                                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                      num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                                      mlp_only_layers=[], max_position_embeddings=256, output_router_logits=False)
    hf = _hf_model(cfg)
    return hf, *_ours(hf, tmp_path)


def test_qwen3_moe_matches_transformers(tmp_path):
    hf, arch, ours = _qwen3_moe(tmp_path)
    _compare(hf, ours, arch)


def test_qwen3_moe_attention_and_mlp_blocks_match_separately(tmp_path):
    """The first decoder layer's attention output and MoE output on the same inputs (attn-only / mlp-only)."""
    hf, arch, ours = _qwen3_moe(tmp_path)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, arch.hidden_size, generator=g)
    seq = SeqInfo.from_lengths([T], "cpu")
    layer_h, layer_o = hf.model.layers[0], ours.model.layers[0]
    pos = torch.arange(T)[None]
    cos_sin = hf.model.rotary_emb(x[None], pos)
    want_attn = layer_h.self_attn(hidden_states=x[None], position_embeddings=cos_sin, attention_mask=_causal(T))[0][0]
    got_attn = layer_o.self_attn(x, seq)
    assert (got_attn - want_attn).abs().max().item() < 2e-4
    want_mlp = layer_h.mlp(x[None])
    want_mlp = (want_mlp[0] if isinstance(want_mlp, tuple) else want_mlp).reshape(T, -1)
    got_mlp = layer_o.mlp(x, seq)
    assert (got_mlp - want_mlp).abs().max().item() < 2e-4


def _causal(n):
    m = torch.full((n, n), float("-inf")).triu(1)
    return m[None, None]


def test_qwen3_moe_router_replay_reproduces_the_recorded_routing(tmp_path):
    """With ``routed_experts`` given, the recorded choices are used whatever the router would pick; feeding a
    forward pass its own choices back must change nothing, feeding other experts must."""
    hf, arch, ours = _qwen3_moe(tmp_path)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, arch.vocab_size, (T,), generator=g)
    seq = SeqInfo.from_lengths([T], "cpu")
    base = ours(ids, seq)
    picked = torch.stack([layer.mlp.last_topk for layer in ours.model.layers], dim=1)      # [T, L, k]
    seq2 = SeqInfo.from_lengths([T], "cpu")
    seq2.routed_experts = picked
    assert torch.allclose(ours(ids, seq2), base, atol=1e-6)
    seq3 = SeqInfo.from_lengths([T], "cpu")
    seq3.routed_experts = (picked + 1) % arch.num_experts
    assert not torch.allclose(ours(ids, seq3), base, atol=1e-4)
    for li, layer in enumerate(ours.model.layers):
        assert torch.equal(layer.mlp.last_topk.long(), seq3.routed_experts[:, li].long())


def test_glm4_moe_matches_transformers(tmp_path):
    cfg = transformers.Glm4MoeConfig(vocab_size=320, hidden_size=64, intermediate_size=160, moe_intermediate_size=48,
                                     num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                     n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                                     first_k_dense_replace=1, norm_topk_prob=True, routed_scaling_factor=1.5,
                                     n_group=1, topk_group=1, use_qk_norm=True, partial_rotary_factor=0.5,
                                     max_position_embeddings=256, attention_bias=True)
    hf = _hf_model(cfg)
    with torch.no_grad():
        for layer in hf.model.layers[1:]:
            layer.mlp.gate.e_score_correction_bias.normal_(0, 0.1)
    arch, ours = _ours(hf, tmp_path)
    _compare(hf, ours, arch)


def test_gpt_oss_matches_transformers(tmp_path):
    cfg = transformers.GptOssConfig(vocab_size=320, hidden_size=64, intermediate_size=48, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_local_experts=4,
                                    num_experts_per_tok=2, sliding_window=16,
                                    layer_types=["sliding_attention", "full_attention"], max_position_embeddings=256,
                                    rope_scaling=None, rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    hf = _hf_model(cfg)
    arch, ours = _ours(hf, tmp_path)
    _compare(hf, ours, arch, atol=5e-4)
