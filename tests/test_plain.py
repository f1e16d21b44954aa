"""The plain implementation against the stored outputs of the reference's own model code, and
against properties each part must have."""

from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

from tests.plain import qwen3_plain as plain

GOLDEN = Path(__file__).parent / "golden"
CASES = {"tiny_a": (plain.tiny_config_a(), 0), "tiny_b": (plain.tiny_config_b(), 7)}


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_matches_reference_outputs(name, tmp_path):
    raw, seed = CASES[name]
    plain.write_random_model(tmp_path, raw, seed)
    gold = load_file(str(GOLDEN / f"{name}.safetensors"))
    cfg, w = plain.read_config(tmp_path), plain.read_weights(tmp_path)
    ours = plain.all_logits(cfg, w, gold["ids"].tolist())
    assert ours.shape == gold["logits"].shape
    assert (ours - gold["logits"]).abs().max().item() < 2e-5


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_sampler_matches_the_reference_samplers_noise_and_tokens(name, tmp_path):
    """The hashed noise (bit for bit) and a continuation sampled at temperature 0.7, as the
    reference's own sampler produced them (stored by tests/golden/make_golden.py)."""
    raw, seed = CASES[name]
    gold = load_file(str(GOLDEN / f"{name}.safetensors"))
    for (sd, ct), row in zip(gold["noise_keys"].tolist(), gold["noise"]):
        assert torch.equal(plain.uniform_noise(sd, ct, raw["vocab_size"]), row)
    plain.write_random_model(tmp_path, raw, seed)
    cfg, w = plain.read_config(tmp_path), plain.read_weights(tmp_path)
    prompt = gold["ids"][:9].tolist()
    assert plain.generate(cfg, w, prompt, 24, temperature=0.7, seed=11) == gold["sampled"].tolist()


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = plain.tiny_config_a(), plain.tiny_config_b()
    for key in ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        assert a[key] != b[key], key
    assert a["num_attention_heads"] // a["num_key_value_heads"] != b["num_attention_heads"] // b["num_key_value_heads"]
    assert b["vocab_size"] & (b["vocab_size"] - 1) and b["hidden_size"] & (b["hidden_size"] - 1)
    assert b["num_attention_heads"] * b["head_dim"] != b["hidden_size"]


def test_rms_norm_part():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    y = plain.rms_norm(x, w, 1e-5)
    expect = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(y, expect, atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    d, theta = 16, 10000.0
    q, k = torch.randn(1, 1, d), torch.randn(1, 1, d)

    def rot(x, p):
        cos, sin = plain.rope_cos_sin(torch.tensor([p]), d, theta, torch.float32)
        return plain.apply_rope(x, cos, sin)

    assert torch.allclose(rot(q, 7).norm(), q.norm(), atol=1e-5)
    s1 = (rot(q, 9) * rot(k, 4)).sum()
    s2 = (rot(q, 25) * rot(k, 20)).sum()
    assert torch.allclose(s1, s2, atol=1e-4)
    assert torch.equal(rot(q, 0), q)


def test_attention_is_causal_and_grouped():
    t, heads, kv, d = 6, 4, 2, 8
    q, k, v = torch.randn(t, heads, d), torch.randn(t, kv, d), torch.randn(t, kv, d)
    out = plain.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0  # the future must not matter
    assert torch.equal(plain.causal_attention(q, k2, v2)[:4], out[:4])
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])  # head 3 reads kv head 1
    w = plain.causal_attention(q, k, v, window=2)
    assert torch.allclose(w[1], out[1]) and not torch.allclose(w[5], out[5])


def test_sampler_noise_and_greedy():
    u = plain.uniform_noise(123, 17, 50)
    assert ((u > 0) & (u < 1)).all() and torch.equal(u, plain.uniform_noise(123, 17, 50))
    assert not torch.equal(u, plain.uniform_noise(123, 18, 50))
    logits = torch.tensor([0.0, 3.0, 3.0, 1.0])
    assert plain.sample_token(logits, 0.0, 0, 0) == 1  # first maximal index
    picks = {plain.sample_token(logits, 1.0, s, 5) for s in range(40)}
    assert picks <= {0, 1, 2, 3} and len(picks) > 1
    assert {plain.sample_token(logits, 1.0, s, 5, top_p=0.4) for s in range(40)} == {1}


def test_generate_recomputes_whole_sequences(tmp_path):
    raw = plain.tiny_config_a()
    plain.write_random_model(tmp_path, raw, 3)
    cfg, w = plain.read_config(tmp_path), plain.read_weights(tmp_path)
    out = plain.generate(cfg, w, [1, 2, 3], 4)
    assert len(out) == 4
    assert out[1] == int(torch.argmax(plain.all_logits(cfg, w, [1, 2, 3, out[0]])[-1]))
