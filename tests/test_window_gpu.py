"""A toy architecture whose layers differ in what they need of the cache: one attends over the last
24 keys only, the other over all of them. The model is Qwen3's parts with a ``window`` on one
mixer, registered in this file; it steps through the step function and generates through the
engine, with and without CUDA graphs, far past the window and past the windowed group's small
pool, against the plain implementation run with the same windows."""

import dataclasses
import json
import random

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.config import Architecture, PartSpec, Qwen3Config, register_architecture, unregister_architecture
from miniserve_b200.engine import LLM, SamplingParams
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from miniserve_b200.models.qwen3 import qwen3_model_spec
from tests.plain import qwen3_plain as plain
from tests.trace_util import check_bfloat16, sharpen_attention

pytestmark = pytest.mark.gpu

WINDOWS = [24, None, 24]
PAGE = 8


def _window_spec(cfg: Qwen3Config):
    spec = qwen3_model_spec(cfg)
    layers = []
    for layer, window in zip(spec.layers, WINDOWS):
        mixer = PartSpec(layer.mixer.kind, dict(layer.mixer.params, window=window))
        layers.append(dataclasses.replace(layer, mixer=mixer))
    return dataclasses.replace(spec, architecture="ToyWindowLM", layers=tuple(layers))


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    register_architecture(Architecture("ToyWindowLM", Qwen3Config.from_dict, _window_spec), replace=True)
    raw = dict(plain.tiny_config_a(), num_hidden_layers=3, architectures=["ToyWindowLM"])
    path = tmp_path_factory.mktemp("toy_window")
    plain.write_random_model(path, raw, seed=21, std=0.05, dtype=torch.bfloat16)
    sharpen_attention(path, 3.0)
    cfg = dict(plain.read_config(path), windows=WINDOWS)
    yield dict(path=path, raw=raw, cfg=cfg, w=plain.read_weights(path), w16=plain.read_weights(path, torch.bfloat16))
    unregister_architecture("ToyWindowLM")


def test_the_windowed_layers_get_a_group_and_a_pool_of_their_own(folder):
    llm = LLM(folder["path"], dtype="bfloat16", kv_pool_tokens=4096, page_size=PAGE, max_running=4, chunked_prefill_size=16)
    d = llm.engine.describe()
    groups = {g["window"]: g for g in d["cache_groups"]}
    assert set(groups) == {24, None} and groups[24]["entries"] == 2 and groups[None]["entries"] == 1
    assert groups[None]["pages"] == 4096 // PAGE
    assert groups[24]["pages"] == 4 * (-(-(24 + 16) // PAGE) + 1)  # four requests' windows and steps, not the whole pool
    assert d["architecture"] == "ToyWindowLM" and d["chunked_prefill_size"] == 16 and d["graph_buckets"] == [1, 2, 4]
    json.dumps(d)  # plain data


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_past_the_window_whole_in_portions_and_decoded(folder, dtype):
    cfg, w = folder["cfg"], folder["w"]
    rng = random.Random(5)
    ids = [rng.randrange(folder["raw"]["vocab_size"]) for _ in range(150)]
    other = [rng.randrange(folder["raw"]["vocab_size"]) for _ in range(90)]
    expect = plain.all_logits(cfg, w, ids)
    _, _, model = load_model(folder["path"], dtype, "cuda:0")
    # the windowed group has 16 pages: a request never holds more than its window and a step there
    from miniserve_b200.cache.manager import group_needs

    pages = [16 if need.window else 64 for need, _ in group_needs(model.entry_caches)[0]]
    cache = CacheManager(model.entry_caches, pages, PAGE, 3, dtype=model.dtype, device=model.device, poison=True,
                         poison_on_free=True, step_tokens=40)
    step = StepFunction(model, cache)
    n = len(ids)
    a = cache.new_request()
    outs, at = [], 0
    for size in (40, 7, 2, 33, 1, 1, 1, 24, 3):  # portions of changing size, single tokens among them
        outs.append(step.run([StepRow(a, ids[at:at + size], range(size))]))
        at += size
    b = cache.new_request()
    while at < n:  # the rest token by token, beside a second request's portions
        rows = [StepRow(a, ids[at:at + 1], [0])]
        done = b.num_tokens
        if done < len(other):
            rows.append(StepRow(b, other[done:done + 5], []))
        outs.append(step.run(rows)[:1])
        at += 1
    step.check_status()
    windowed = [g for g in cache.groups if g.need.window][0]
    assert windowed.allocator.num_used <= 2 * (-(-(24 + 5) // PAGE) + 1)  # what the window has passed came back
    cache.release(a)
    cache.release(b)
    assert cache.is_idle()
    got = torch.cat(outs).cpu()
    err = (got - expect).abs().max(dim=1).values
    if dtype == "float32":
        assert err.max().item() <= 5e-5 * max(1.0, expect.abs().max().item()), f"position {int(err.argmax())}: {err.max().item():.3e}"
    else:
        rough = (plain.all_logits(cfg, folder["w16"], ids).float() - expect).abs().max(dim=1).values
        check_bfloat16(err, (rough.max().item(), rough.mean().item()), "windowed steps")
    # without the window the same tokens give other logits: the window is really applied
    full = plain.all_logits(dict(cfg, windows=None), w, ids)
    assert (full[60:] - expect[60:]).abs().max().item() > (100 if dtype == "float32" else 5) * err.max().item()


@pytest.mark.parametrize("dtype, cuda_graph", [("float32", False), ("float32", True), ("bfloat16", True), ("bfloat16", False)])
def test_generation_far_past_the_window_with_and_without_graphs(folder, dtype, cuda_graph):
    cfg, w, raw = folder["cfg"], folder["w"], folder["raw"]
    rng = random.Random(9)
    prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(n)] for n in (45, 3, 70, 17, 30)]
    # a pool of 40 pages of 8 tokens holds two or three of these requests at a time: pages are used again
    llm = LLM(folder["path"], dtype=dtype, kv_pool_tokens=320, page_size=PAGE, max_running=4, chunked_prefill_size=16,
              cuda_graph=cuda_graph)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=80))
    eng = llm.engine
    assert eng.cache.is_idle() and eng.scheduler.num_preemptions > 0  # the full group's pool was short
    if cuda_graph:
        assert eng.graphs.replayed_launches > 0
    for p, o in zip(prompts, outs):
        assert len(o) == 80
        if dtype == "float32":
            assert o == plain.generate(cfg, w, p, 80)
        else:
            # teacher-forced: every chosen token is the plain implementation's best up to what rounding to
            # bfloat16 moves logits by (measured on this very sequence: two logits that far apart may swap)
            seq = list(p) + o[:40]
            exact = plain.all_logits(cfg, w, seq)
            rough = plain.all_logits(cfg, folder["w16"], seq).float()
            slack = 2 * (rough - exact).abs().max().item()
            for i, t in enumerate(o[:40]):
                logits = exact[len(p) + i - 1]
                assert (logits.max() - logits[t]).item() <= slack, f"token {t} at {len(p) + i}: beyond {slack:.3f}"
