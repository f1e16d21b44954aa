"""The engine at the layer sizes of a real checkpoint (Qwen3-0.6B: hidden 1024, 16 query heads,
8 kv heads, head size 128, intermediate 3072, vocabulary 151,936, tied head), with fewer layers and
random weights, against the plain implementation: the sizes at which the serving kernels (tensor-core
attention for head size 128, the weight-streaming decode product, the two-stage sampler) run."""

import random

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.config import preset
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from tests.plain import qwen3_plain as plain
from tests.trace_util import bfloat16_noise, check_bfloat16, sharpen_attention

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    raw = preset("0.6b")
    raw["num_hidden_layers"] = 3
    path = tmp_path_factory.mktemp("qwen3_06b_shapes")
    plain.write_random_model(path, raw, seed=5, dtype=torch.bfloat16)
    sharpen_attention(path, 2.0)
    rng = random.Random(4)
    ids = [rng.randrange(raw["vocab_size"]) for _ in range(200)]
    cfg, w = plain.read_config(path), plain.read_weights(path)
    expect = plain.all_logits(cfg, w, ids)
    return dict(path=path, raw=raw, ids=ids, expect=expect)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_whole_in_portions_and_decoded(real, dtype):
    ids, expect = real["ids"], real["expect"]
    _, _, model = load_model(real["path"], dtype, "cuda:0")
    cache = CacheManager(model.entry_caches, 40, 16, 4, dtype=model.dtype, device=model.device, poison=True)
    step = StepFunction(model, cache)
    n = len(ids)
    # whole
    rc = cache.new_request()
    whole = step.run([StepRow(rc, ids, range(n))])
    cache.release(rc)
    # a portion of 150, then 18 tokens one by one beside a second request's portions, then the rest in one portion
    a, b = cache.new_request(), cache.new_request()
    outs = [step.run([StepRow(a, ids[:150], range(150))])]
    for i in range(150, 168):
        rows = [StepRow(a, ids[i:i + 1], [0])]
        if i < 160:
            rows.append(StepRow(b, ids[(i - 150) * 20:(i - 149) * 20], []))
        outs.append(step.run(rows)[:1])
    outs.append(step.run([StepRow(a, ids[168:], range(n - 168)), StepRow(b, ids[:3], [])])[:n - 168])
    step.check_status()
    cut = torch.cat(outs)
    cache.release(a)
    cache.release(b)
    assert cache.is_idle()
    scale = max(1.0, expect.abs().max().item())
    for name, got in (("whole", whole), ("cut", cut)):
        err = (got.cpu() - expect).abs().max(dim=1).values
        if dtype == "float32":
            assert err.max().item() <= 5e-5 * scale, f"{name}: position {int(err.argmax())} off by {err.max().item():.3e}"
        else:
            noise = bfloat16_noise(real["path"], {"x": ids}, {"x": expect})
            check_bfloat16(err, noise, name)
    if dtype == "float32":
        assert torch.equal(whole, cut)  # bit-identical however the tokens were cut and batched


def test_real_vocabulary_sampling_matches_the_plain_sampler(real):
    _, _, model = load_model(real["path"], "float32", "cuda:0")
    cache = CacheManager(model.entry_caches, 8, 16, 2, dtype=model.dtype, device=model.device)
    step = StepFunction(model, cache)
    rc = cache.new_request()
    logits = step.run([StepRow(rc, real["ids"][:40], [38, 39])])
    from miniserve_b200.sampling import Sampler

    sampler = Sampler(model.device, model.spec.vocab_size)
    greedy = sampler.sample(logits).tolist()
    assert greedy == torch.argmax(logits, -1).tolist()
    got = sampler.sample(logits, temperatures=[0.8, 1.0], top_ps=[1.0, 1.0], seeds=[7, 9], counters=[39, 40]).tolist()
    for r in range(2):
        assert got[r] == plain.sample_token(logits[r].cpu(), [0.8, 1.0][r], [7, 9][r], [39, 40][r])
    cache.release(rc)


def test_wide_hidden_size_runs_the_tcgen05_products_and_their_epilogues(tmp_path, monkeypatch):
    """A hidden size of 2,048 with this package's tcgen05 kernels forced for every product with more
    than 16 rows: the q|k|v product then carries the per-head norm, the rotation and the cache write
    in its epilogue and the gate|up product SiLU * up. Whole, in portions and decoded, against the
    plain implementation."""
    from miniserve_b200 import ops

    monkeypatch.setattr(ops, "TC_GEMM", "1")
    raw = dict(plain.tiny_config_b(), hidden_size=2048, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
               intermediate_size=512, vocab_size=777, num_hidden_layers=2, tie_word_embeddings=False)
    plain.write_random_model(tmp_path, raw, seed=9, std=0.02, dtype=torch.bfloat16)
    rng = random.Random(8)
    ids = [rng.randrange(raw["vocab_size"]) for _ in range(330)]
    cfg, w = plain.read_config(tmp_path), plain.read_weights(tmp_path)
    expect = plain.all_logits(cfg, w, ids)
    _, _, model = load_model(tmp_path, "bfloat16", "cuda:0")
    assert ops.qkv_fused_ok(torch.empty(300, 2048, device="cuda", dtype=torch.bfloat16), model.layers[0].mixer.w_qkv, 4, 2, 128, 128,
                            True, model.layers[0].mixer.w_q_norm, model.layers[0].mixer.w_k_norm)
    cache = CacheManager(model.entry_caches, 48, 16, 4, dtype=model.dtype, device=model.device, poison=True)
    step = StepFunction(model, cache)
    n = len(ids)
    rc = cache.new_request()
    whole = step.run([StepRow(rc, ids, range(n))])
    cache.release(rc)
    a, b = cache.new_request(), cache.new_request()
    outs = [step.run([StepRow(a, ids[:257], range(257))])]
    for i in range(257, 270):
        outs.append(step.run([StepRow(a, ids[i:i + 1], [0]), StepRow(b, ids[(i - 257) * 19:(i - 256) * 19], [])])[:1])
    outs.append(step.run([StepRow(b, ids[:40], []), StepRow(a, ids[270:], range(n - 270))])[:n - 270])
    step.check_status()
    cut = torch.cat(outs)
    cache.release(a)
    cache.release(b)
    assert cache.is_idle()
    noise = bfloat16_noise(tmp_path, {"x": ids}, {"x": expect})
    for name, got in (("whole", whole), ("cut", cut)):
        check_bfloat16((got.cpu() - expect).abs().max(dim=1).values, noise, name)
