"""Configurations at the edges of what the kernels take: widths, feed-forward sizes and
vocabularies that are no multiple of 8, head sizes from 16 to 256 in steps of 16, one to seven
heads in a group, pages of 4 to 64 tokens. Each model is stepped whole, in portions beside
another request's decoded tokens, and one token at a time, in float32 and in bfloat16, against
the plain implementation."""

import random

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from tests.plain import qwen3_plain as plain
from tests.trace_util import bfloat16_noise, check_bfloat16, sharpen_attention

pytestmark = pytest.mark.gpu


def _config(hidden, inter, vocab, layers, nq, nkv, d, theta=10000.0, eps=1e-6, tie=True):
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=hidden, intermediate_size=inter, vocab_size=vocab,
                num_hidden_layers=layers, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
                rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tie, max_position_embeddings=512,
                hidden_act="silu")


CASES = {
    "nothing_in_eights": (_config(100, 130, 333, 2, 5, 5, 16), 16),
    "head_48_one_kv_head": (_config(72, 200, 1001, 2, 3, 1, 48, theta=5e5, eps=1e-5, tie=False), 8),
    "head_80_pages_of_32": (_config(256, 520, 2048, 2, 8, 2, 80), 32),
    "head_112_seven_heads": (_config(64, 96, 130, 3, 7, 7, 112, eps=1e-4), 64),
    "head_256": (_config(128, 384, 777, 1, 2, 2, 256, tie=False), 16),
    "width_36_pages_of_4": (_config(36, 52, 97, 2, 3, 3, 32), 4),
}


@pytest.fixture(scope="module", params=sorted(CASES))
def model_folder(request, tmp_path_factory):
    raw, page = CASES[request.param]
    path = tmp_path_factory.mktemp(request.param)
    plain.write_random_model(path, raw, 3, std=0.05, dtype=torch.bfloat16)
    sharpen_attention(path)
    rng = random.Random(5)
    seqs = {k: [rng.randrange(raw["vocab_size"]) for _ in range(n)] for k, n in (("a", 150), ("b", 90))}
    cfg, w = plain.read_config(path), plain.read_weights(path, torch.float32)
    expect = {k: plain.all_logits(cfg, w, ids) for k, ids in seqs.items()}
    return dict(path=path, page=page, seqs=seqs, expect=expect)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoded_tokens_of_an_odd_configuration(model_folder, dtype):
    seqs, expect, page = model_folder["seqs"], model_folder["expect"], model_folder["page"]
    a, b = seqs["a"], seqs["b"]
    _, _, model = load_model(model_folder["path"], dtype, "cuda:0")
    cache = CacheManager(model.entry_caches, -(-150 // page) + -(-90 // page) + 1, page, 2, dtype=model.dtype,
                         device=model.device, poison=True)
    step = StepFunction(model, cache)
    ra, rb = cache.new_request(), cache.new_request()
    got = {"a": [], "b": []}

    def run(rows):
        """rows: (name, request, first token, count); every token's logits are wanted"""
        out = step.run([StepRow(rc, seqs[k][s:s + n], list(range(n))) for k, rc, s, n in rows]).cpu()
        at = 0
        for k, _, s, n in rows:
            assert len(got[k]) == s
            got[k] += list(out[at:at + n])
            at += n

    run([("a", ra, 0, 118)])
    run([("a", ra, 118, 1), ("b", rb, 0, 2)])
    run([("a", ra, 119, 1), ("b", rb, 2, 17)])
    run([("a", ra, 120, 1), ("b", rb, 19, 63)])
    for i in range(8):
        run([("a", ra, 121 + i, 1), ("b", rb, 82 + i, 1)])
    run([("a", ra, 129, 21)])
    step.check_status()
    cache.release(ra)
    cache.release(rb)
    assert cache.is_idle()
    errors = torch.cat([(torch.stack(got[k]) - expect[k]).abs().max(dim=1).values for k in ("a", "b")])
    if dtype == "float32":
        scale = max(1.0, max(e.abs().max().item() for e in expect.values()))
        over = (errors > 3e-5 * scale).nonzero().flatten().tolist()  # positions of a (0..149), then of b (150..239)
        assert not over, f"worst {errors.max().item():.3e} at {int(errors.argmax())}; over the tolerance at {over}"
    else:
        check_bfloat16(errors, bfloat16_noise(model_folder["path"], seqs, expect), "an odd configuration")
