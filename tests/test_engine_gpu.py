"""The engine on the GPU: greedy generation through the entry point, long decoding, the first
tokens of a sequence, sampling, cache pressure, and CUDA graphs, against the plain implementation."""

import random

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.engine import LLM, SamplingParams
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from tests.plain import qwen3_plain as plain
from tests.trace_util import bfloat16_noise, check_bfloat16, sharpen_attention

pytestmark = pytest.mark.gpu

CASES = {"tiny_a": (plain.tiny_config_a(), 0, 16), "tiny_b": (plain.tiny_config_b(), 7, 8)}


@pytest.fixture(scope="module", params=sorted(CASES))
def folder(request, tmp_path_factory):
    raw, seed, page = CASES[request.param]
    path = tmp_path_factory.mktemp(request.param)
    plain.write_random_model(path, raw, seed, std=0.05, dtype=torch.bfloat16)
    sharpen_attention(path)
    return dict(path=path, raw=raw, page=page, cfg=plain.read_config(path), w=plain.read_weights(path))


def _prompts(raw, lengths, seed):
    rng = random.Random(seed)
    return [[rng.randrange(raw["vocab_size"]) for _ in range(n)] for n in lengths]


def _margins_ok(cfg, w, prompt, tokens, eps):
    """Teacher-forced: each chosen token's plain logit is within eps of the plain maximum
    (the rule of the reference's tests/anchor.py:43-64)."""
    seq = list(prompt)
    for t in tokens:
        logits = plain.all_logits(cfg, w, seq)[-1]
        assert (logits.max() - logits[t]).item() <= eps, f"token {t} at {len(seq)} is not (nearly) the best"
        seq.append(t)


@pytest.mark.parametrize("dtype, cuda_graph", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_entry_point(folder, dtype, cuda_graph):
    raw = folder["raw"]
    prompts = _prompts(raw, [5, 17, 33, 1, 9], 1)
    llm = LLM(folder["path"], dtype=dtype, kv_pool_tokens=1024, page_size=folder["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=cuda_graph)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=12))
    assert llm.engine.cache.is_idle()
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        if dtype == "float32":
            assert o == plain.generate(folder["cfg"], folder["w"], p, 12)
        else:
            _margins_ok(folder["cfg"], folder["w"], p, o, eps=0.05)


def test_generation_under_cache_pressure_equals_each_request_alone(folder):
    raw = folder["raw"]
    prompts = _prompts(raw, [30, 12, 25, 7, 40, 18], 3)
    params = SamplingParams(max_new_tokens=20)
    roomy = LLM(folder["path"], dtype="float32", kv_pool_tokens=2048, page_size=folder["page"], max_running=6,
                chunked_prefill_size=16, cuda_graph=False)
    expect = roomy.generate(prompts, params)
    tight = LLM(folder["path"], dtype="float32", kv_pool_tokens=128, page_size=folder["page"], max_running=6,
                chunked_prefill_size=16, cuda_graph=False)
    got = tight.generate(prompts, params)
    assert tight.engine.scheduler.num_preemptions > 0, "the pool was meant to run out"
    assert got == expect  # bit-equal float32 logits make the tokens equal whatever was batched or recomputed
    assert tight.engine.cache.is_idle()
    assert got[0] == plain.generate(folder["cfg"], folder["w"], prompts[0], 20)


def test_temperature_sampling_is_seeded_and_matches_the_plain_sampler(folder):
    raw = folder["raw"]
    prompts = _prompts(raw, [9, 40, 3], 4)
    params = [SamplingParams(10, temperature=0.7, seed=11), SamplingParams(10, temperature=0.0),
              SamplingParams(10, temperature=1.2, top_p=0.9, seed=5)]
    llm = LLM(folder["path"], dtype="float32", kv_pool_tokens=1024, page_size=folder["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=True)
    outs = llm.generate(prompts, params)
    again = llm.generate(prompts[::-1], params[::-1])[::-1]  # other rows beside it, other pages: same tokens
    assert outs == again
    assert outs[0] == plain.generate(folder["cfg"], folder["w"], prompts[0], 10, temperature=0.7, seed=11)
    assert outs[1] == plain.generate(folder["cfg"], folder["w"], prompts[1], 10)
    other_seed = llm.generate(prompts[:1], SamplingParams(10, temperature=0.7, seed=12))[0]
    assert other_seed != outs[0]


def test_stop_token_ends_a_request_and_is_kept(folder):
    prompt = _prompts(folder["raw"], [8], 6)[0]
    free = plain.generate(folder["cfg"], folder["w"], prompt, 8)
    llm = LLM(folder["path"], dtype="float32", kv_pool_tokens=256, page_size=folder["page"], cuda_graph=False)
    out = llm.generate([prompt], SamplingParams(8, stop_token_ids=frozenset({free[3]})))[0]
    assert out == free[:free.index(free[3]) + 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folder, dtype):
    """Three hundred tokens one by one against the whole sequence at once; and positions 0, 1, 2."""
    raw = folder["raw"]
    n = 300
    ids = _prompts(raw, [n], 8)[0]
    expect = plain.all_logits(folder["cfg"], folder["w"], ids)
    _, _, model = load_model(folder["path"], dtype, "cuda:0")
    cache = CacheManager(model.entry_caches, -(-n // folder["page"]) + 1, folder["page"], 2, dtype=model.dtype,
                         device=model.device, poison=True)
    step = StepFunction(model, cache)
    rc = cache.new_request()
    rows = [step.run([StepRow(rc, ids[i:i + 1], [0])]) for i in range(n)]
    step.check_status()
    got = torch.cat(rows).cpu()
    # float32: only the order of sums differs. bfloat16: as near to the float32 truth as the plain
    # implementation is when it runs in bfloat16 itself on these tokens
    scale = max(1.0, expect.abs().max().item())
    err = (got - expect).abs().max(dim=1).values
    if dtype == "float32":
        tol = 3e-5 * scale
        assert err.max().item() <= tol, f"worst position {int(err.argmax())}: {err.max().item():.3e}"
    else:
        noise = bfloat16_noise(folder["path"], {"x": ids}, {"x": expect})
        check_bfloat16(err, noise, "decoding one by one")
        tol = 2 * noise[0]
    cache.release(rc)
    # the first tokens as a step of their own, in pages that were just used by someone else
    rc = cache.new_request()
    first = step.run([StepRow(rc, ids[:3], [0, 1, 2])]).cpu()
    assert (first - expect[:3]).abs().max().item() <= tol
    cache.release(rc)
    assert cache.is_idle()


def test_a_graph_replays_rightly_after_later_captures_and_a_trimmed_allocator(folder):
    """A capture empties the allocator's cache, and so may anyone: a graph captured earlier must
    hold no address of memory that went back to the allocator (everything its pass allocated
    comes from the graphs' own pool)."""
    raw = folder["raw"]
    llm = LLM(folder["path"], dtype="float32", kv_pool_tokens=1024, page_size=folder["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=True)
    first = _prompts(raw, [6, 11], 21)
    lengths = [5, 14]  # two requests decode together, then one alone: the graphs for 2 rows and for 1
    outs = llm.generate(first, [SamplingParams(max_new_tokens=n) for n in lengths])
    assert len(llm.engine.graphs._graphs) >= 2
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    scribble = [torch.full((1 << 18,), float("nan"), device="cuda:0") for _ in range(8)]  # takes what was given back
    second = _prompts(raw, [9, 4], 22)
    outs += llm.generate(second, [SamplingParams(max_new_tokens=n) for n in lengths])  # the first graphs again
    del scribble
    for p, o, n in zip(first + second, outs, lengths * 2):
        assert o == plain.generate(folder["cfg"], folder["w"], p, n)


def test_graphs_captured_at_the_start_in_every_mode(folder):
    """Every batch bucket in all three sampling modes captured before any request, one after the
    other (each capture empties the allocator's cache under the ones before it), then generation."""
    raw = folder["raw"]
    llm = LLM(folder["path"], dtype="float32", kv_pool_tokens=1024, page_size=folder["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=True)
    captured = llm.engine.capture_graphs(("greedy", "temperature", "top_p"))
    assert captured == 3 * len(llm.engine.graphs.buckets)
    assert llm.engine.cache.is_idle()
    prompts = _prompts(raw, [7, 19, 3], 31)
    greedy = llm.generate(prompts, SamplingParams(max_new_tokens=9))
    for p, o in zip(prompts, greedy):
        assert o == plain.generate(folder["cfg"], folder["w"], p, 9)
    sampled = llm.generate(prompts[:1], SamplingParams(9, temperature=0.8, seed=3))[0]
    assert sampled == plain.generate(folder["cfg"], folder["w"], prompts[0], 9, temperature=0.8, seed=3)
    nucleus = llm.generate(prompts[:1], SamplingParams(9, temperature=0.8, top_p=0.8, seed=3))[0]
    eager = LLM(folder["path"], dtype="float32", kv_pool_tokens=1024, page_size=folder["page"], max_running=4,
                chunked_prefill_size=24, cuda_graph=False)
    assert nucleus == eager.generate(prompts[:1], SamplingParams(9, temperature=0.8, top_p=0.8, seed=3))[0]
    assert len(llm.engine.graphs._graphs) == captured  # nothing was captured again


def test_a_long_request_decodes_through_the_graph_for_its_class_of_context_length(tmp_path):
    """A request past 8,192 tokens replays the decode graph captured for long contexts (its keys shared
    out among as many CTAs as fit the GPU, merged through scratch memory), a short one beside it the graph
    for short contexts afterwards; the tokens are those of the same engine without graphs."""
    raw = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 2,
           "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 256, "vocab_size": 701, "rms_norm_eps": 1e-6,
           "rope_theta": 1000000.0, "tie_word_embeddings": True, "hidden_act": "silu", "max_position_embeddings": 16384}
    plain.write_random_model(tmp_path, raw, seed=5, dtype=torch.bfloat16)
    rng = random.Random(3)
    prompts = [[rng.randrange(701) for _ in range(n)] for n in (8200, 60)]
    params = [SamplingParams(max_new_tokens=5), SamplingParams(max_new_tokens=12)]
    outs = {}
    for graphs in (True, False):
        llm = LLM(tmp_path, dtype="bfloat16", kv_pool_tokens=16384, page_size=16, max_running=4, cuda_graph=graphs)
        outs[graphs] = llm.generate(prompts, params)
        assert llm.engine.cache.is_idle()
        if graphs:
            classes = {key[2] for key in llm.engine.graphs._graphs}
            assert classes == {0, 8192}, classes
    assert outs[True] == outs[False]
