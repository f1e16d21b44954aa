"""The scheduler's decisions and the engine loop, on the host, against a stand-in step function.

The stand-in (after the idea of the reference's ``_ToyModel``, tests/test_engine.py:481-559)
keeps, per pool slot, which (token, position) was written there; every step re-reads each
row's whole history through its block table, checks that positions are 0..n-1, and emits
logits that are a deterministic function of that history. A wrong page, a stale slot or a
token run twice shows up as a failed check or a different output.
"""

import hashlib
import random

import pytest
import torch

from miniserve_b200.cache import CacheManager, OutOfBlocks
from miniserve_b200.engine.engine import Engine
from miniserve_b200.engine.request import InvalidTransition, Request, RequestState, SamplingParams
from miniserve_b200.engine.scheduler import Scheduler
from miniserve_b200.parts import PagedKV
from miniserve_b200.parts.decoder import EntryCache
from tests.plain import qwen3_plain as plain

VOCAB = 37


def _cache(pages, page=4, max_requests=64):
    return CacheManager([EntryCache(0, PagedKV(1, 8)), EntryCache(1, PagedKV(1, 8))], pages, page, max_requests)


class ToyStep:
    def __init__(self, cache):
        self.cache = cache
        self.store = {}
        self.status = torch.zeros(1, dtype=torch.int32)
        self.max_tokens_seen = 0

    @staticmethod
    def logits_of(history):
        h = hashlib.sha256(repr(tuple(history)).encode()).digest()
        g = torch.Generator().manual_seed(int.from_bytes(h[:8], "little") % (2 ** 63))
        return torch.randn(VOCAB, generator=g)

    def run(self, rows, prev_tokens=None):
        rows = list(rows)
        for r in rows:
            if r.fill_from is not None:  # a token the host has not read back yet: it is on the "device"
                assert len(r.tokens) == 1 and prev_tokens is not None
                r.tokens = [int(prev_tokens[r.fill_from])]
        self.cache.reserve([(r.cache, len(r.tokens)) for r in rows])
        self.max_tokens_seen = max(self.max_tokens_seen, sum(len(r.tokens) for r in rows))
        out = []
        for r in rows:
            table = r.cache.tables[0]
            end = table.num_tokens
            start = end - len(r.tokens)
            for i, tok in enumerate(r.tokens):
                self.store[table.slot(start + i)] = (tok, start + i)
            history = []
            for p in range(end):
                tok, pos = self.store[table.slot(p)]
                assert pos == p, f"slot of position {p} holds position {pos}"
                history.append(tok)
            for w in r.want:
                out.append(self.logits_of(history[:start + w + 1]))
        return torch.stack(out) if out else torch.zeros((0, VOCAB))


    def reset_after_fault(self):
        self.status.zero_()
        self.resets = getattr(self, "resets", 0) + 1


class ToySampler:
    def sample(self, logits, temperatures=None, top_ps=None, seeds=None, counters=None, stream=None):
        n = logits.shape[0]
        if temperatures is None:
            return torch.argmax(logits, -1).to(torch.int32)
        return torch.tensor([plain.sample_token(logits[i], temperatures[i], seeds[i], counters[i], top_ps[i])
                             for i in range(n)], dtype=torch.int32)


def _engine(pages, page=4, chunk=8, max_running=64, overlap=False, **kw):
    cm = _cache(pages, page, max_running)
    eng = Engine(None, cache=cm, step_fn=ToyStep(cm), sampler=ToySampler(), max_running=max_running,
                 chunked_prefill_size=chunk, cuda_graph=False, overlap=overlap, **kw)
    return eng


def _alone(prompt, params, seed):
    """What the request produces when it runs alone: the whole sequence recomputed per token."""
    seq, out = list(prompt), []
    for _ in range(params.max_new_tokens):
        tok = plain.sample_token(ToyStep.logits_of(seq), params.temperature, seed, len(seq), params.top_p)
        out.append(tok)
        seq.append(tok)
        if tok in params.stop_token_ids:
            break
    return out


# ------------------------------------------------------------------ requests
def test_state_machine():
    r = Request(0, [1, 2], SamplingParams(4))
    with pytest.raises(InvalidTransition):
        r.transition(RequestState.DECODE)
    r.transition(RequestState.PREFILL)
    r.transition(RequestState.WAITING)  # preempted between portions
    r.transition(RequestState.PREFILL)
    r.transition(RequestState.DECODE)
    r.transition(RequestState.WAITING)  # preempted while decoding
    r.transition(RequestState.ABORTED)
    with pytest.raises(InvalidTransition):
        r.transition(RequestState.WAITING)
    with pytest.raises(ValueError):
        Request(1, [], SamplingParams(1))


@pytest.mark.parametrize("kw", [dict(max_new_tokens=0), dict(max_new_tokens=1, temperature=-1.0),
                                dict(max_new_tokens=1, top_p=0.0), dict(max_new_tokens=1, top_p=1.5),
                                dict(max_new_tokens=1, seed=2 ** 32)])
def test_sampling_params_are_validated(kw):
    with pytest.raises(ValueError):
        SamplingParams(**kw)


def test_token_slice_spans_prompt_and_output():
    r = Request(0, [1, 2, 3], SamplingParams(8), output_ids=[7, 8])
    assert r.token_slice(0, 5) == [1, 2, 3, 7, 8] and r.token_slice(2, 2) == [3, 7] and r.token_slice(3, 2) == [7, 8]
    assert r.seq_len == 5 and r.max_len == 11


# ------------------------------------------------------------------ decisions
def test_oversized_request_is_rejected_when_added():
    s = Scheduler(_cache(4), chunked_prefill_size=8)
    s.add(Request(0, [1] * 10, SamplingParams(6)))  # 16 tokens = 4 pages: fits
    with pytest.raises(ValueError, match="pool holds 16"):
        s.add(Request(1, [1] * 10, SamplingParams(7)))


def test_chunked_steps_decode_first_then_portions_in_admission_order():
    eng = _engine(pages=64, chunk=8)
    a = eng.add_request(list(range(1, 12)), SamplingParams(3))   # 11 tokens
    b = eng.add_request(list(range(1, 6)), SamplingParams(3))    # 5 tokens
    p1 = eng.step()
    assert [(r.request.rid, r.start, r.count) for r in p1.rows] == [(0, 0, 8)] and p1.phase == "prefill"
    assert a.state is RequestState.PREFILL and b.state is RequestState.WAITING and not a.output_ids
    p2 = eng.step()  # rest of a (3), then b admitted with what is left of the budget (5)
    assert [(r.request.rid, r.start, r.count) for r in p2.rows] == [(0, 8, 3), (1, 0, 5)]
    assert a.state is RequestState.DECODE and b.state is RequestState.DECODE
    assert len(a.output_ids) == 1 and len(b.output_ids) == 1
    c = eng.add_request(list(range(1, 20)), SamplingParams(2))
    p3 = eng.step()  # two decode rows first, six tokens of c
    assert p3.phase == "mixed" and p3.num_decode == 2
    assert [(r.request.rid, r.start, r.count) for r in p3.rows] == [(0, 11, 1), (1, 5, 1), (2, 0, 6)]
    assert p3.num_tokens == 8
    while eng.has_unfinished:
        eng.step()
    assert eng.cache.is_idle()


def test_admission_stops_at_the_first_request_that_does_not_fit():
    eng = _engine(pages=6, page=4, chunk=64)
    eng.add_request([1] * 13, SamplingParams(2))  # needs ceil(14/4) = 4 pages
    eng.add_request([1] * 9, SamplingParams(2))   # needs 3: does not fit beside the first
    eng.add_request([1] * 2, SamplingParams(2))   # would fit, but must not skip ahead
    plan = eng.step()
    assert [r.request.rid for r in plan.rows] == [0]
    assert [r.rid for r in eng.scheduler.waiting] == [1, 2]


def test_whole_prefill_mode_keeps_phases_apart():
    eng = _engine(pages=64, chunk=0, max_prefill_tokens=10)
    eng.add_request([1] * 7, SamplingParams(2))
    eng.add_request([1] * 3, SamplingParams(2))
    eng.add_request([1] * 4, SamplingParams(2))  # over the 10-token budget of the first prefill step
    p1 = eng.step()
    assert p1.phase == "prefill" and [r.count for r in p1.rows] == [7, 3]
    p2 = eng.step()
    assert p2.phase == "prefill" and [r.request.rid for r in p2.rows] == [2]
    p3 = eng.step()
    assert p3.phase == "decode" and p3.num_decode == 3
    big = _engine(pages=64, chunk=0, max_prefill_tokens=4)
    big.add_request([1] * 9, SamplingParams(1))
    assert big.step().rows[0].count == 9  # the first request is admitted even over the budget


def test_pages_run_out_newest_is_preempted_oldest_never_and_output_is_unchanged():
    prompts = [[3 + i] * 6 for i in range(4)]
    params = SamplingParams(10)
    eng = _engine(pages=10, page=4, chunk=32)  # 40 tokens of pool for 4 x 16 tokens of demand
    reqs = [eng.add_request(p, params) for p in prompts]
    oldest = reqs[0]
    steps = 0
    while eng.has_unfinished:
        plan = eng.step()
        assert plan is not None and oldest not in plan.preempted
        for victim in plan.preempted:
            assert victim.state is RequestState.WAITING and victim.cache is None
        eng.cache.check_invariants()
        steps += 1
        assert steps < 500
    assert eng.scheduler.num_preemptions > 0 and oldest.num_preemptions == 0
    assert max(r.num_preemptions for r in reqs) > 0
    for r, p in zip(reqs, prompts):
        assert r.output_ids == _alone(p, params, r.seed)
    assert eng.cache.is_idle()


def test_shortest_job_first_orders_admission_and_picks_the_longest_to_preempt():
    """``schedule_policy="sjf"``: least remaining work first (prompt tokens still to compute plus tokens that
    may still be generated), equals in arrival order, and still no skipping past one that does not fit."""
    eng = _engine(pages=64, chunk=64, max_running=2, schedule_policy="sjf")
    a = eng.add_request([1] * 9, SamplingParams(4))    # 13 to go
    b = eng.add_request([1] * 3, SamplingParams(30))   # 33
    c = eng.add_request([1] * 5, SamplingParams(2))    # 7
    d = eng.add_request([1] * 4, SamplingParams(3))    # 7, after c
    plan = eng.step()
    assert [r.request.rid for r in plan.rows] == [c.rid, d.rid]  # two may run
    while not (c.is_done and d.is_done):
        eng.step()
    assert [r.request.rid for r in eng.step().rows][-1] in (a.rid, b.rid) and a.state is not RequestState.WAITING
    while eng.has_unfinished:
        eng.step()
    assert eng.cache.is_idle()
    # the one with least work does not fit: nothing behind it is tried
    eng = _engine(pages=6, page=4, chunk=64, schedule_policy="sjf")
    eng.add_request([1] * 13, SamplingParams(8))   # runs first (alone in the queue), holds 4 of 6 pages
    eng.step()
    eng.add_request([1] * 9, SamplingParams(1))    # 10 to go, needs 3 pages: does not fit
    eng.add_request([1] * 2, SamplingParams(20))   # 22 to go, would fit
    assert [r.request.rid for r in eng.step().rows] == [0]
    assert sorted(r.rid for r in eng.scheduler.waiting) == [1, 2]
    # when pages run out the request with most left to do goes, never the oldest
    eng = _engine(pages=10, page=4, chunk=32, schedule_policy="sjf")
    reqs = [eng.add_request([3 + i] * 6, SamplingParams(n)) for i, n in enumerate((10, 4, 10, 6))]
    victims = []
    while eng.has_unfinished:
        plan = eng.step()
        victims += [v.rid for v in plan.preempted]
        assert reqs[0] not in plan.preempted
        eng.cache.check_invariants()
    assert victims and victims[0] == 2  # most remaining work among all but the oldest (ties: the newest)
    for r in reqs:
        assert r.output_ids == _alone(r.prompt_ids, r.params, r.seed)
    with pytest.raises(ValueError, match="unknown schedule policy"):
        _engine(pages=8, schedule_policy="cache")


def test_preempted_request_reruns_prompt_plus_output():
    eng = _engine(pages=5, page=4, chunk=32)
    a = eng.add_request([1] * 7, SamplingParams(8))
    b = eng.add_request([2] * 7, SamplingParams(8))
    seen = []
    while eng.has_unfinished:
        plan = eng.step()
        seen += [(r.request.rid, r.start, r.count) for r in plan.rows]
    assert b.num_preemptions > 0
    reruns = [x for x in seen if x[0] == b.rid and x[1] == 0]
    assert len(reruns) >= 2 and reruns[1][2] > 7  # the second prefill of b runs prompt + kept output


def test_abort_gives_everything_back():
    eng = _engine(pages=16, chunk=8)
    a = eng.add_request([1] * 5, SamplingParams(50))
    b = eng.add_request([2] * 5, SamplingParams(3))
    eng.step()
    eng.step()
    eng.abort(a.rid)
    assert a.state is RequestState.ABORTED and a.cache is None
    while eng.has_unfinished:
        eng.step()
    assert b.state is RequestState.FINISHED and eng.cache.is_idle()
    eng.abort(12345)  # unknown ids are ignored


def test_overlap_launches_before_it_reads_back():
    eng = _engine(pages=32, chunk=8, overlap=True)
    a = eng.add_request([4, 5, 6], SamplingParams(4))
    eng.step()  # launches the prefill; nothing is read back yet
    assert a.output_ids == [-1] and a.num_pending == 1 and a.state is RequestState.DECODE and a.ready_ids == []
    plan = eng.step()  # launches the first decode step with a placeholder input, reads the prefill's token
    assert plan.phase == "decode" and a.num_pending == 1 and len(a.ready_ids) == 1
    while eng.has_unfinished:
        eng.step()
    assert a.output_ids == _alone([4, 5, 6], SamplingParams(4), a.seed) and a.num_pending == 0
    assert eng.cache.is_idle()


def test_overlap_drops_the_token_sampled_past_a_stop():
    free_run = _alone([4, 5, 6], SamplingParams(8), 0)
    stop = free_run[2]
    eng = _engine(pages=32, chunk=8, overlap=True)
    r = eng.add_request([4, 5, 6], SamplingParams(8, stop_token_ids=frozenset({stop})))
    other = eng.add_request([9, 9], SamplingParams(8))
    while eng.has_unfinished:
        eng.step()
    assert r.output_ids == free_run[:free_run.index(stop) + 1] and r.num_pending == 0
    assert other.output_ids == _alone([9, 9], SamplingParams(8), other.seed)
    assert eng.cache.is_idle()


def test_stop_token_is_kept_and_ends_the_request():
    eng = _engine(pages=16, chunk=8)
    free_run = _alone([4, 5, 6], SamplingParams(6), 0)
    stop = free_run[2]
    r = eng.add_request([4, 5, 6], SamplingParams(6, stop_token_ids=frozenset({stop})))
    while eng.has_unfinished:
        eng.step()
    first = free_run.index(stop)
    assert r.output_ids == free_run[:first + 1]


# ------------------------------------------------------------------ randomised load
@pytest.mark.parametrize("policy", ["fcfs", "sjf"])
@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("pages, chunk", [(8, 3), (16, 3), (64, 3), (8, 2048), (16, 2048), (64, 2048), (8, 0), (64, 0)])
def test_random_load_equals_each_request_alone(pages, chunk, overlap, policy):
    preemptions = 0
    for seed in range(6):
        rng = random.Random(1000 * pages + seed)
        eng = _engine(pages=pages, page=4, chunk=chunk, max_running=6, seed=seed, max_prefill_tokens=24, overlap=overlap,
                      schedule_policy=policy)
        specs = []
        for i in range(12):
            prompt = [rng.randrange(VOCAB) for _ in range(rng.randint(1, 14))]
            temp = rng.choice([0.0, 0.0, 0.7, 1.3])
            params = SamplingParams(rng.randint(1, 12), frozenset({rng.randrange(VOCAB)}), temp,
                                    rng.choice([1.0, 0.8]) if temp else 1.0)
            if pages * 4 < len(prompt) + params.max_new_tokens:
                continue
            specs.append((prompt, params))
        reqs, pending, steps = [], list(specs), 0
        while pending or eng.has_unfinished:
            for _ in range(rng.randint(0, 3)):  # requests arrive while others run
                if pending:
                    reqs.append(eng.add_request(*pending.pop(0)))
            if eng.has_unfinished:
                plan = eng.step()
                assert plan is not None or eng.overlap
                if chunk and plan is not None:
                    assert plan.num_tokens <= max(chunk, plan.num_decode)
                eng.cache.check_invariants()
            steps += 1
            assert steps < 5000, "no progress"
        for r, (prompt, params) in zip(reqs, specs):
            assert r.state is RequestState.FINISHED
            assert r.output_ids == _alone(prompt, params, r.seed), (pages, chunk, seed, r.rid)
        assert eng.cache.is_idle()
        preemptions += eng.scheduler.num_preemptions
    if pages == 8:
        assert preemptions > 0, "the small pool must actually run out of pages"


@pytest.mark.parametrize("overlap", [False, True])
def test_a_raised_status_word_ends_the_step_once_and_the_engine_goes_on(overlap):
    """A kernel that caught a fault raises the status word; the engine reports it once, frees nothing
    twice, puts the word back and can be used again."""
    from miniserve_b200.engine.step import StepError

    eng = _engine(pages=32, overlap=overlap)
    prompts = [[1, 2, 3, 4, 5], [6, 7, 8]]
    reqs = [eng.add_request(p, SamplingParams(max_new_tokens=6)) for p in prompts]
    eng.step()
    eng.step_fn.status[0] = 31  # as a kernel would, from the device
    with pytest.raises(StepError, match="31"):
        while eng.has_unfinished:
            eng.step()
    assert eng.step_fn.resets == 1 and int(eng.step_fn.status[0]) == 0
    for r in reqs:  # the caller gives up on what was running; nothing is released twice
        if not r.is_done:
            eng.abort(r.rid)
    eng._inflight = None
    eng.cache.check_invariants()
    assert eng.cache.is_idle() and not eng.scheduler.has_unfinished
    out = eng.generate(prompts, SamplingParams(max_new_tokens=4))
    assert [len(o) for o in out] == [4, 4] and eng.cache.is_idle()


def test_generate_leaves_nothing_behind_when_a_prompt_is_refused():
    eng = _engine(pages=8, page=4)  # 32 tokens of cache
    ok, too_long = [1, 2, 3], list(range(30))
    with pytest.raises(ValueError, match="pool holds"):
        eng.generate([ok, too_long], SamplingParams(max_new_tokens=8))
    assert not eng.has_unfinished and not eng.requests and not eng.scheduler.waiting
    with pytest.raises(ValueError, match="sampling parameters"):
        eng.generate([ok, ok], [SamplingParams(max_new_tokens=1)])
    assert eng.generate([ok], SamplingParams(max_new_tokens=3)) == [_alone(ok, SamplingParams(max_new_tokens=3), 0)]


def test_engine_describes_itself():
    eng = _engine(pages=16, chunk=8, max_running=4)
    d = eng.describe() if eng.model is not None else None
    assert d is None  # the stand-in engine has no model; the GPU tests check the description of a real one


def test_overlap_with_every_running_request_preempted_is_no_stall():
    """With overlap, a request preempted while its newest token is still on the device cannot be admitted
    again before that token is read back. If nothing else can run, the step that reads it back launches
    nothing; that is progress, not a stall (a model with a windowed cache group beside a full one, whose
    full group is short, gets there)."""

    class CountingStep(ToyStep):
        def run(self, rows, prev_tokens=None):
            rows = list(rows)
            self.cache.reserve([(r.cache, len(r.tokens)) for r in rows])
            out = [self.logits_of((id(r.cache) % 1000, r.cache.num_tokens, w)) for r in rows for w in r.want]
            for r in rows:
                self.cache.trim(r.cache)
            return torch.stack(out) if out else torch.zeros((0, VOCAB))

    entries = [EntryCache(0, PagedKV(1, 8, window=24)), EntryCache(1, PagedKV(1, 8)), EntryCache(2, PagedKV(1, 8, window=24))]
    cm = CacheManager(entries, [24, 40], 8, 4, step_tokens=16)
    eng = Engine(None, cache=cm, step_fn=CountingStep(cm), sampler=ToySampler(), max_running=4, chunked_prefill_size=16,
                 cuda_graph=False, overlap=True)
    rng = random.Random(9)
    prompts = [[rng.randrange(VOCAB) for _ in range(n)] for n in (45, 3, 70, 17, 30)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=80))
    assert [len(o) for o in outs] == [80] * 5 and eng.scheduler.num_preemptions > 0
    cm.check_invariants()
    assert cm.is_idle()


def test_graph_batch_sizes_and_key_splits_of_a_decode_step():
    """The padded batch sizes that decode graphs are captured for, and how many CTAs share a request's keys
    (host decisions: ``engine/graphs.py`` graph_buckets, ``ops/attention_bf16.py`` choose_splits)."""
    from miniserve_b200.engine.graphs import graph_buckets
    from miniserve_b200.ops.attention_bf16 import choose_splits

    assert graph_buckets(1) == [1] and graph_buckets(8) == [1, 2, 4, 8] and graph_buckets(9) == [1, 2, 4, 8, 9]
    assert graph_buckets(24) == [1, 2, 4, 8, 16, 24] and graph_buckets(40) == [1, 2, 4, 8, 16, 24, 32, 40]
    assert graph_buckets(64) == [1, 2, 4, 8, 16, 24, 32, 48, 64]
    # clusters of n CTAs that a B200 holds at a time with head size 128 (a cluster stays inside one GPC)
    resident = {2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33}.__getitem__
    assert choose_splits(8, 8, None, 148, resident) == 4
    assert choose_splits(6, 8, None, 148) == 6 and choose_splits(6, 8, None, 148, resident) == 5  # 48 clusters of 6 where 45 fit
    assert choose_splits(12, 8, None, 148, resident) == 2  # 96 clusters of 3 where 93 fit
    assert choose_splits(1, 8, None, 148, resident) == 8 and choose_splits(4, 8, None, 148, resident) == 8
    assert choose_splits(1, 8, 200, 148, resident) == 2  # never fewer than 128 keys to a split
    assert choose_splits(64, 8, None, 148, resident) == 1 and choose_splits(1, 8, 4000, 148) == 16
    # long contexts: as many CTAs as fit the GPU at once; a few more than a cluster's 8 splits stay a cluster
    assert choose_splits(1, 8, 8192, 148, resident) == 32 and choose_splits(1, 8, 131072, 148, resident) == 37
    assert choose_splits(2, 8, 32768, 148, resident) == 18 and choose_splits(4, 8, 32768, 148, resident) == 8
    from miniserve_b200.engine.graphs import length_class
    assert [length_class(n) for n in (1, 8191, 8192, 40000, 131072, 10 ** 6)] == [0, 0, 8192, 32768, 131072, 131072]
