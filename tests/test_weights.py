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


def test_loader_joins_stacks_in_place_and_follows_rename_and_split_rules(tmp_path):
    """A checkpoint that names a tensor differently and stores q, k and v as one matrix is read
    through rules (data of the architecture); the parts' stacks come back joined, equal to the
    concatenation of their pieces."""
    from miniserve_b200.config import TensorRule

    raw = preset("tiny-a")
    write_model_folder(tmp_path, raw, seed=3)
    model = _model(raw)
    decls, stacks = model.weight_decls(), model.weight_stacks()
    assert stacks["model.layers.0.self_attn.qkv_proj.weight"] == tuple(
        f"model.layers.0.self_attn.{n}_proj.weight" for n in "qkv")
    plain_load = load_weights(tmp_path, decls, torch.bfloat16, "cpu")
    joined = load_weights(tmp_path, decls, torch.bfloat16, "cpu", stacks=stacks)
    for name, pieces in stacks.items():
        assert name in joined and not any(p in joined for p in pieces)
        assert torch.equal(joined[name], torch.cat([plain_load[p] for p in pieces]))
    model.bind(joined)  # the parts take the joined tensors as they are
    assert model.layers[0].mixer.w_qkv.data_ptr() == joined["model.layers.0.self_attn.qkv_proj.weight"].data_ptr()
    again = _model(raw)
    again.bind(plain_load)
    assert torch.equal(again.layers[1].feed_forward.w_gate_up, model.layers[1].feed_forward.w_gate_up)
    # the same checkpoint stored the other way: the final norm under another name, q|k|v of layer 1 as one matrix
    tensors = load_file(str(tmp_path / "model.safetensors"))
    tensors["final_layernorm.scale"] = tensors.pop("model.norm.weight")
    pre = "model.layers.1.self_attn."
    fused = torch.cat([tensors.pop(pre + f"{n}_proj.weight") for n in "qkv"])
    tensors[pre + "fused_qkv.weight"] = fused
    other = tmp_path / "renamed"
    other.mkdir()
    save_file(tensors, str(other / "model.safetensors"))
    rows = [decls[pre + f"{n}_proj.weight"].shape[0] for n in "qkv"]
    rules = (TensorRule.rename("final_layernorm.scale", "model.norm.weight"),
             TensorRule.split(pre + "fused_qkv.weight", *[(pre + f"{n}_proj.weight", r) for n, r in zip("qkv", rows)]))
    mapped = load_weights(other, decls, torch.bfloat16, "cpu", rules=rules, stacks=stacks)
    assert set(mapped) == set(joined) and all(torch.equal(mapped[k], joined[k]) for k in joined)
    with pytest.raises(CheckpointMismatch) as ei:  # without the rules the same folder does not match, in one error
        load_weights(other, decls, torch.bfloat16, "cpu", stacks=stacks)
    assert "model.norm.weight" in ei.value.missing and pre + "fused_qkv.weight" in ei.value.unexpected
    bad = (rules[0], TensorRule.split(pre + "fused_qkv.weight", (pre + "q_proj.weight", rows[0]), (pre + "k_proj.weight", 1)))
    with pytest.raises(CheckpointMismatch) as ei:
        load_weights(other, decls, torch.bfloat16, "cpu", rules=bad, stacks=stacks)
    assert any("cannot be cut" in w for w in ei.value.wrong_shape) and pre + "v_proj.weight" in ei.value.missing


def test_random_weights_fill_stacks_with_the_values_the_pieces_would_have():
    raw = preset("tiny-b")
    model = _model(raw)
    decls, stacks = model.weight_decls(), model.weight_stacks()
    alone = random_tensors(decls, 9)
    joined = random_tensors(decls, 9, stacks=stacks)
    for name, pieces in stacks.items():
        assert torch.equal(joined[name], torch.cat([alone[p] for p in pieces]))
    assert torch.equal(joined["lm_head.weight"], alone["lm_head.weight"])
