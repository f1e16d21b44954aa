import json

import pytest

from miniserve_b200.config import (PRESETS, Architecture, ModelSpec, PartSpec, Qwen3Config, RunEntry,
                                   architecture_of, architectures, load_config_dict, preset, register_architecture,
                                   resolve, unregister_architecture)
from miniserve_b200.models.qwen3 import qwen3_model_spec


def test_qwen3_config_reads_the_reference_keys():
    raw = preset("tiny-b")
    cfg = Qwen3Config.from_dict(raw)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (96, 3, 6, 1)
    assert cfg.head_dim == 32 and cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and not cfg.tie_word_embeddings
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_head_dim_and_tie_defaults():
    raw = preset("tiny-a")
    del raw["head_dim"], raw["tie_word_embeddings"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == 64 // 4 and cfg.tie_word_embeddings is False


@pytest.mark.parametrize("patch, exc", [
    (dict(rope_scaling={"type": "yarn"}), NotImplementedError),
    (dict(hidden_act="gelu"), NotImplementedError),
    (dict(num_key_value_heads=3), ValueError),
    (dict(head_dim=15), ValueError),
    (dict(vocab_size=0), ValueError),
])
def test_unsupported_configs_are_refused(patch, exc):
    raw = preset("tiny-a")
    raw.update(patch)
    with pytest.raises(exc):
        Qwen3Config.from_dict(raw)


def test_missing_key_is_named():
    raw = preset("tiny-a")
    del raw["rms_norm_eps"]
    with pytest.raises(KeyError, match="rms_norm_eps"):
        Qwen3Config.from_dict(raw)


def test_registry_resolves_by_architecture_name(tmp_path):
    assert "Qwen3ForCausalLM" in architectures()
    (tmp_path / "config.json").write_text(json.dumps(preset("tiny-a")))
    arch, cfg, spec = resolve(load_config_dict(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config) and isinstance(spec, ModelSpec)
    with pytest.raises(ValueError, match="unknown architecture"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ValueError, match="architectures"):
        architecture_of({})
    with pytest.raises(FileNotFoundError):
        load_config_dict(tmp_path / "nope")


def test_registering_another_architecture():
    arch = Architecture("ToyLM", lambda raw: raw, lambda cfg: None)
    register_architecture(arch)
    try:
        with pytest.raises(ValueError, match="already"):
            register_architecture(arch)
        assert architecture_of({"architectures": ["ToyLM"]}) is arch
    finally:
        unregister_architecture("ToyLM")


def test_model_spec_carries_every_constant_as_a_parameter():
    cfg = Qwen3Config.from_dict(preset("tiny-b"))
    spec = qwen3_model_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    mixer = spec.layers[1].mixer
    assert mixer.kind == "gqa_attention" and mixer["heads"] == 6 and mixer["kv_heads"] == 1 and mixer["head_dim"] == 32
    assert mixer["qk_norm_eps"] == 1e-5 and mixer["position"]["theta"] == 1e6
    assert spec.layers[0].feed_forward["intermediate"] == 224
    assert spec.head["tied"] is False and spec.final_norm["eps"] == 1e-5
    assert spec.layers[2].prefix == "model.layers.2."


def test_run_order_is_validated():
    cfg = Qwen3Config.from_dict(preset("tiny-a"))
    spec = qwen3_model_spec(cfg)
    kw = {f: getattr(spec, f) for f in ("architecture", "hidden_size", "vocab_size", "embedding", "layers",
                                         "final_norm", "head", "final_norm_prefix")}
    ModelSpec(run_order=(RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)), **kw)  # twice, shared: fine
    with pytest.raises(ValueError):
        ModelSpec(run_order=(RunEntry(5),), **kw)
    with pytest.raises(ValueError):
        ModelSpec(run_order=(RunEntry(0, cache_of=0),), **kw)


def test_presets_are_the_published_shapes():
    assert set(PRESETS) >= {"tiny-a", "tiny-b", "0.6b", "8b", "32b"}
    c = Qwen3Config.from_dict(preset("0.6b"))
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.tie_word_embeddings) == (28, 1024, 16, 8, 128, 3072, 151936, True)
    with pytest.raises(ValueError):
        preset("70b")
    assert PartSpec("x", {"a": 1})["a"] == 1
