"""Prompt and mixed steps replayed from CUDA graphs (``engine/graphs.py``, ``StepGraphs``) against the
same steps launched eagerly: the same bits, whichever way a step of a recurring shape (tokens, rows,
wanted logits, decoding rows) shares its tokens among its rows. Two step functions over the same model
and caches of their own run the same steps; one has the graphs. One exception to "the same bits": in
bfloat16 the decoding rows of a captured step have their keys split as inside a decode graph (by the
number of rows, not by their lengths), so their sums are taken in another order, and the products of a
padded step run over more rows, which may change their rounding; from the first such step on the two
sides are compared within bfloat16's resolution instead. float32 stays exact throughout.

The model has head size 128, so the steps run through the tcgen05 attention (kept out of the graphs
and called between them with each step's own geometry), the decode attention for the single-token
rows at the front of a mixed step, and the tensor-core or library products."""

import random

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.engine.graphs import StepGraphs
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

RAW = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 320, "num_hidden_layers": 3, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 736, "vocab_size": 1931, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "tie_word_embeddings": False, "hidden_act": "silu", "max_position_embeddings": 4096,
}
PAGE = 16


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    path = tmp_path_factory.mktemp("step_graphs")
    plain.write_random_model(path, RAW, seed=21, dtype=torch.bfloat16)
    return path


class Pair:
    """An eager step function and one with graphs, over caches of their own, fed the same steps."""

    def __init__(self, folder, dtype, pages=80, slots=6, arena_ints=1 << 16, **graph_args):
        _, _, self.model = load_model(folder, dtype, "cuda:0")
        self.caches = [CacheManager(self.model.entry_caches, pages, PAGE, slots, dtype=self.model.dtype,
                                    device=self.model.device, poison=True) for _ in range(2)]
        self.eager = StepFunction(self.model, self.caches[0])
        self.graphed = StepFunction(self.model, self.caches[1], arena_ints=arena_ints)
        graph_args.setdefault("capture_every", 0)  # the tests want every capture at once,
        graph_args.setdefault("sightings", 2)      # at a shape's second sighting
        self.graphs = StepGraphs(self.graphed, indices_cap=pages + 2 * slots + 4, **graph_args)
        self.graphed.graphs = self.graphs
        self.requests: dict[str, tuple] = {}
        self.rng = random.Random(9)
        self.exact = True  # until a bfloat16 step with decoding rows has been captured

    def step(self, rows):
        """rows: (request name, number of new tokens, wanted places). The same bits from both, or it fails."""
        built = ([], [])
        for name, count, want in rows:
            if name not in self.requests:
                self.requests[name] = tuple(c.new_request() for c in self.caches)
            tokens = [self.rng.randrange(RAW["vocab_size"]) for _ in range(count)]
            for side in range(2):
                built[side].append(StepRow(self.requests[name][side], tokens, want))
        want = self.eager.run(built[0]).clone()
        captures = self.graphs.captures
        got = self.graphed.run(built[1]).clone()
        key = self.graphs._key(built[1])
        ran_in_a_graph = key is not None and key in self.graphs._shapes
        if self.model.dtype == torch.bfloat16 and ran_in_a_graph:
            if self.graphs.captures > captures and len(built[1][0].tokens) == 1:
                self.exact = False
            if key[0] != sum(len(r.tokens) for r in built[1]):  # padded: the products ran over more rows
                self.exact = False
        assert got.shape == want.shape
        off = (got - want).abs().max().item() if got.numel() else 0.0
        if self.exact:
            assert torch.equal(got, want), f"step {rows}: off by {off:.3e}"
        else:
            assert off <= 2.0 ** -6 * max(1.0, want.abs().max().item()), f"step {rows}: off by {off:.3e}"
        return got

    def end(self, name):
        for cache, rc in zip(self.caches, self.requests.pop(name)):
            cache.release(rc)

    def finish(self):
        for name in list(self.requests):
            self.end(name)
        self.eager.check_status()
        self.graphed.check_status()
        assert all(c.is_idle() for c in self.caches)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recurring_shapes_replay_with_the_same_bits_however_the_rows_share_the_tokens(folder, dtype):
    p = Pair(folder, dtype)
    g = p.graphs
    assert g.enabled
    # (96 tokens, 1 row, 1 wanted): eager, captured, replayed; each time a new request on other pages
    for i in range(3):
        p.step([(f"a{i}", 96, (95,))])
    assert g.captures == 1 and sum(h.uses for h in g._shapes.values()) == 2
    # the same shape further into the requests: the prefix grows, pages differ, a request continues on used pages
    p.step([("a0", 96, (0,))])
    p.end("a1")
    p.step([("a2", 96, (40,))])
    p.step([("b", 96, (7,))])
    assert g.captures == 1
    # (40 tokens, 3 rows, 2 wanted) shared out in different ways: decode rows at the front, then portions
    p.step([("a0", 1, (0,)), ("a2", 1, (0,)), ("c", 38, ())])
    p.step([("a0", 1, (0,)), ("a2", 9, (8,)), ("c", 30, ())])
    p.step([("a0", 1, ()), ("b", 2, (0, 1)), ("c", 37, ())])
    assert g.captures == 2
    # the same numbers without a decoding row at the front: a shape of its own, whose attention stays inside the graph
    p.step([("a0", 20, (19,)), ("a2", 10, (3,)), ("b", 10, ())])
    p.step([("a0", 5, (4,)), ("a2", 30, (3,)), ("b", 5, ())])
    p.step([("b", 2, ()), ("c", 2, (0, 1)), ("a0", 36, ())])
    assert g.captures == 3
    assert all(len(h.pieces) == 1 for h in g._shapes.values()), "with head size 128 every step is one graph"
    # decode-only steps and tiny steps are not taken
    before = sum(h.uses for h in g._shapes.values())
    p.step([("a0", 1, (0,)), ("b", 1, (0,))])
    p.step([("a0", 1, (0,)), ("b", 1, (0,))])
    p.step([("c", 3, (2,))])
    p.step([("c", 3, (2,))])
    assert sum(h.uses for h in g._shapes.values()) == before and g.captures == 3
    p.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_any_length_meet_a_padded_shape(folder, dtype):
    """Steps are rounded up to the next multiple of 32 tokens (64 beyond 256, 128 beyond 512) by a row of
    their own on the page outside the allocator: lengths of one bucket replay one graph, and the real rows'
    results are those of the unpadded step (the same bits in float32)."""
    assert [StepGraphs.padded(n) for n in (16, 33, 256, 257, 512, 513, 2048)] == [32, 64, 256, 320, 512, 640, 2048]
    p = Pair(folder, dtype)
    g = p.graphs
    for i, n in enumerate((70, 75, 90, 65, 96)):  # 96 itself is a shape without padding, seen once
        p.step([(f"a{i}", n, (n - 1,))])
    assert g.captures == 1 and sum(h.uses for h in g._shapes.values()) == 3
    (key,) = g._shapes
    assert key == (96, 2, 1, 0)  # 96 tokens in two rows: the prompt and the padding
    # portions behind a prefix, and a decoding row in front of a portion: padded alike
    p.step([("a0", 33, (32,))])
    p.step([("a1", 50, (49,))])
    p.step([("a0", 1, (0,)), ("a2", 20, (19,))])
    p.step([("a1", 1, (0,)), ("a3", 25, (24,))])
    p.step([("a0", 1, (0,)), ("a2", 28, (27,))])
    assert g.captures == 3 and set(g._shapes) == {(96, 2, 1, 0), (64, 2, 1, 0), (32, 3, 2, 1)}
    # a long padding row: 257 tokens run as 320
    for name in ("a0", "a1", "a2", "a3", "a4"):
        p.end(name)
    for i in range(3):
        p.step([(f"b{i}", 257, (256,))])
    assert (320, 2, 1, 0) in g._shapes
    p.finish()
    # without padding every length is a shape of its own
    q = Pair(folder, dtype, pad=False)
    for i, n in enumerate((70, 75, 90, 65)):
        q.step([(f"a{i}", n, (n - 1,))])
    assert q.graphs.captures == 0
    q.finish()


def test_attention_kept_out_of_the_graphs_when_its_launch_follows_the_rows(folder, monkeypatch):
    """Without the tcgen05 attention kernel (whose plan can live on the device) attention is called between
    the graphs, with every step's own rows."""
    from miniserve_b200 import ops

    monkeypatch.setattr(ops, "TC_ATTENTION", False)
    p = Pair(folder, "bfloat16")
    g = p.graphs
    for i in range(3):
        p.step([(f"a{i}", 96, (95,))])
    p.step([("a0", 1, (0,)), ("a2", 9, (8,)), ("c", 30, ())])
    p.step([("a0", 1, ()), ("b", 2, (0, 1)), ("c", 37, ())])
    p.step([("a0", 1, (0,)), ("b", 20, (0,)), ("c", 19, ())])
    assert g.captures == 2 and sum(h.uses for h in g._shapes.values()) == 4
    assert all(len(h.pieces) == 2 * RAW["num_hidden_layers"] + 1 for h in g._shapes.values())
    p.finish()


def test_shapes_beyond_the_limit_are_dropped_and_captured_again(folder):
    p = Pair(folder, "bfloat16", max_shapes=2)
    g = p.graphs
    sizes = (48, 64, 80)
    for round_ in range(3):
        for n in sizes:
            for rep in range(2):
                name = f"r{round_}_{n}_{rep}"
                p.step([(name, n, (n - 1,))])
                p.end(name)
        assert len(g._shapes) == 2
    assert g.captures >= 5  # every size was captured, dropped, and captured again
    p.finish()


def test_captures_are_spaced_out(folder):
    p = Pair(folder, "bfloat16", capture_every=40)  # prompts alone keep an eighth of that distance: 5 steps
    g = p.graphs
    def once(n, i):
        p.step([(f"t{n}_{i}", n, (n - 1,))])
        p.end(f"t{n}_{i}")
    once(48, 0)
    once(48, 1)
    assert g.captures == 1  # the second sighting, and nothing was captured lately
    for i in range(5):
        once(64, i)
    assert g.captures == 1  # seen five times, but the last capture is less than six steps back
    once(64, 5)
    assert g.captures == 2
    p.finish()


def test_an_arena_that_has_to_grow_drops_the_graphs(folder):
    p = Pair(folder, "bfloat16", pages=160, arena_ints=1024)
    g = p.graphs
    for i in range(3):
        p.step([(f"s{i}", 64, (63,))])
    assert g.captures == 1
    generation = p.graphed.arena_generation
    for i in range(3):  # needs more room than the arena has: it moves, and what was captured is void
        p.step([(f"l{i}", 600, (599,))])
    assert p.graphed.arena_generation > generation
    p.step([("s0", 64, (1,))])
    p.step([("s1", 64, (1,))])
    p.finish()


def test_a_model_with_a_part_that_reads_the_rows_on_the_host_is_left_alone(folder):
    from miniserve_b200.parts.mlp import SwiGLU

    p = Pair(folder, "bfloat16")
    assert p.model.shape_static
    try:
        SwiGLU.shape_static = False
        assert not p.model.shape_static
        graphs = StepGraphs(p.graphed, indices_cap=100)
        assert not graphs.enabled
        rc = p.caches[1].new_request()
        assert graphs.run([StepRow(rc, [1] * 64, (63,))]) is None and graphs.run([StepRow(rc, [1] * 64, (63,))]) is None
        p.caches[1].release(rc)
    finally:
        SwiGLU.shape_static = True
    # nor is a step taken whose products outweigh its launches by far
    heavy = StepGraphs(p.graphed, indices_cap=100, max_step_flops=1e6)
    rc = p.caches[1].new_request()
    assert heavy.enabled and heavy.run([StepRow(rc, [1] * 64, (63,))]) is None and heavy.run([StepRow(rc, [1] * 64, (63,))]) is None
    p.caches[1].release(rc)
    p.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_with_prompts_in_equal_portions_replays_graphs_and_gives_the_same_tokens(folder, dtype):
    from miniserve_b200.engine import LLM, SamplingParams

    rng = random.Random(2)
    prompts = [[rng.randrange(RAW["vocab_size"]) for _ in range(n)] for n in (200, 150, 96, 333, 64)]
    params = SamplingParams(max_new_tokens=10)
    outs = {}
    for graphs in (False, True):
        llm = LLM(folder, dtype=dtype, kv_pool_tokens=2048, page_size=PAGE, max_running=4, chunked_prefill_size=48,
                  cuda_graph=graphs)
        outs[graphs] = llm.generate(prompts, params)
        assert llm.engine.cache.is_idle()
        if graphs:
            g = llm.engine.step_fn.graphs
            assert llm.engine.describe()["step_graphs"] and g.captures >= 1 and g.replayed_launches > 0
            # and once more over the same engine: the shapes are there already
            captures = g.captures
            assert llm.generate(prompts, params) == outs[True]
            assert g.captures <= captures + 2
        else:
            assert llm.engine.step_fn.graphs is None
    assert outs[True] == outs[False]


def test_prompt_shapes_captured_ahead_are_replayed_by_the_first_requests(folder):
    from miniserve_b200.engine import LLM, SamplingParams

    rng = random.Random(4)
    prompts = [[rng.randrange(RAW["vocab_size"]) for _ in range(n)] for n in (17, 90, 131, 250, 300)]
    params = SamplingParams(max_new_tokens=4)
    eager = LLM(folder, dtype="float32", kv_pool_tokens=2048, page_size=PAGE, max_running=4, cuda_graph=False)
    llm = LLM(folder, dtype="float32", kv_pool_tokens=2048, page_size=PAGE, max_running=4)
    g = llm.engine.step_fn.graphs
    captured = llm.engine.capture_graphs(prompt_tokens=320)
    assert g.captures == 9 and set(g._shapes) == {(n, 2, 1, 0) for n in (32, 64, 96, 128, 160, 192, 224, 256, 320)}
    assert captured == g.captures + len(llm.engine.graphs._graphs) and llm.engine.cache.is_idle()
    outs = [llm.generate([p], params)[0] for p in prompts]
    assert g.captures == 9 and sum(h.uses for h in g._shapes.values()) == 9 + len(prompts)
    assert outs == [eager.generate([p], params)[0] for p in prompts]
