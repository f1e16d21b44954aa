import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from miniserve_b200.config import preset, resolve
from miniserve_b200.parts import DecoderModel
from miniserve_b200.weights import CheckpointMismatch, load_weights, random_tensors, write_model_folder
from tests.plain import qwen3_plain as plain


def _model(raw, dtype=torch.bfloat16):
    _, _, spec = resolve(raw)
    return DecoderModel(spec, dtype, "cpu")


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_declared_names_and_shapes_are_the_checkpoints(name):
    raw = preset(name)
    decls = _model(raw).weight_decls()
    assert {k: tuple(v.shape) for k, v in decls.items()} == plain.expected_shapes(raw)


def test_random_folder_round_trip(tmp_path):
    raw = preset("tiny-b")
    write_model_folder(tmp_path, raw, seed=5)
    assert json.loads((tmp_path / "config.json").read_text())["hidden_size"] == 96
    stored = load_file(str(tmp_path / "model.safetensors"))
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    model = _model(raw)
    w = load_weights(tmp_path, model.weight_decls(), torch.bfloat16, "cpu")
    assert set(w) == set(model.weight_decls())
    assert torch.equal(w["model.norm.weight"], stored["model.norm.weight"])
    w32 = load_weights(tmp_path, model.weight_decls(), torch.float32, "cpu")
    assert w32["lm_head.weight"].dtype == torch.float32
    assert torch.equal(w32["lm_head.weight"], stored["lm_head.weight"].float())
    # same seed, same model; another seed, another model
    again = random_tensors(model.weight_decls(), 5)
    assert all(torch.equal(again[k], stored[k]) for k in stored)
    assert not torch.equal(random_tensors(model.weight_decls(), 6)["lm_head.weight"], stored["lm_head.weight"])
    norm = stored["model.layers.0.input_layernorm.weight"].float()
    assert abs(norm.mean().item() - 1.0) < 0.1 and stored["lm_head.weight"].float().std().item() < 0.03


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    raw = preset("tiny-a")
    write_model_folder(tmp_path, raw, seed=1)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.layers.1.self_attn.q_norm.weight"]
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(8, 8, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    model = _model(raw)
    with pytest.raises(ValueError) as ei:
        load_weights(tmp_path, model.weight_decls(), torch.bfloat16, "cpu")
    err = ei.value
    assert isinstance(err, CheckpointMismatch)
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.layers.1.self_attn.q_norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.wrong_shape) == 1 and "k_proj" in err.wrong_shape[0] and "(8, 8)" in err.wrong_shape[0]
    msg = str(err)
    for needle in ("up_proj", "q_norm", "rotary_emb", "k_proj", "missing", "unexpected", "wrong shape"):
        assert needle in msg


def test_tied_checkpoint_may_ship_a_duplicate_head(tmp_path):
    raw = preset("tiny-a")
    write_model_folder(tmp_path, raw, seed=1)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(tmp_path / "model.safetensors"))
    model = _model(raw)
    with pytest.raises(CheckpointMismatch):
        load_weights(tmp_path, model.weight_decls(), torch.bfloat16, "cpu")
    w = load_weights(tmp_path, model.weight_decls(), torch.bfloat16, "cpu", ignorable={"lm_head.weight"})
    assert "lm_head.weight" not in w


def test_untied_model_needs_its_head(tmp_path):
    raw = preset("tiny-b")
    write_model_folder(tmp_path, raw, seed=1)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    del tensors["lm_head.weight"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointMismatch, match="lm_head"):
        load_weights(tmp_path, _model(raw).weight_decls(), torch.bfloat16, "cpu")


def test_no_safetensors_is_a_file_error(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(preset("tiny-a")))
    with pytest.raises(FileNotFoundError):
        load_weights(tmp_path, _model(preset("tiny-a")).weight_decls(), torch.bfloat16, "cpu")


def test_stored_32bit_tensor_stays_when_declared_so(tmp_path):
    from miniserve_b200.parts import WeightDecl

    save_file({"a": torch.ones(3, dtype=torch.float32), "b": torch.ones(3, dtype=torch.float32),
               "t": torch.arange(4, dtype=torch.int64)}, str(tmp_path / "model.safetensors"))
    decls = {"a": WeightDecl((3,)), "b": WeightDecl((3,), precision="stored"), "t": WeightDecl((4,), precision="int32")}
    w = load_weights(tmp_path, decls, torch.bfloat16, "cpu")
    assert w["a"].dtype == torch.bfloat16 and w["b"].dtype == torch.float32 and w["t"].dtype == torch.int32
