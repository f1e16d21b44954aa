"""Replay through bin/trace_run, in 32-bit and in bfloat16, compared with the plain implementation:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size down to two tokens; and mixed, up to four live requests, portions of
some beside decoded tokens of others, in a pool so small that pages are used again."""

import random

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.trace_util import Trace, bfloat16_noise, check_bfloat16, plain_logits, run_trace, sharpen_attention

pytestmark = pytest.mark.gpu

CONFIGS = {
    "tiny_a": dict(raw=plain.tiny_config_a(), seed=0, ids_seed=1, lengths=[5, 17, 33, 70], page=16),
    "tiny_b": dict(raw=plain.tiny_config_b(), seed=7, ids_seed=2, lengths=[1, 9, 40, 64, 100], page=8),
}
# what "beyond rounding" means here: float32 differs from the plain implementation only by the
# order of sums (a few 1e-7 on logits of size one); bfloat16 may be as far from the float32
# truth as the plain implementation itself is when it runs in bfloat16 on the same tokens
TOL_F32 = 3e-5


def _sequences(case):
    rng = random.Random(case["ids_seed"])
    vocab = case["raw"]["vocab_size"]
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(case["lengths"])}


def _build_trace(seqs):
    tr = Trace()
    tags = {}
    # 1. each request alone and whole
    for rid, ids in seqs.items():
        tr.step([(f"w-{rid}", ids, "all")], end=[f"w-{rid}"])
        tags[f"w-{rid}"] = rid
    # 2. most of it in one step, the last 32 tokens (or all but the first) one by one
    for rid, ids in seqs.items():
        if len(ids) < 2:
            continue
        head = max(1, len(ids) - 32)
        name = f"d-{rid}"
        tags[name] = rid
        tr.step([(name, ids[:head], "last")])
        for p in range(head, len(ids)):
            tr.step([(name, ids[p:p + 1], [0])], end=[name] if p == len(ids) - 1 else [])
    # 3. portions of changing size, down to two tokens
    sizes = [7, 2, 24, 3, 16, 2, 5, 32, 2, 9]
    for rid, ids in seqs.items():
        name = f"c-{rid}"
        tags[name] = rid
        i = k = 0
        while i < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - i)
            k += 1
            tr.step([(name, ids[i:i + n], "all")], end=[name] if i + n == len(ids) else [])
            i += n
    # 4. mixed: up to four live, portions of some beside decoded tokens of others; finished
    #    requests free their pages, which the next arrivals take over
    order = list(seqs)
    rng = random.Random(5)
    waiting = [(f"m{j}-{rid}", rid) for j in range(2) for rid in order]
    live: dict[str, list] = {}
    while waiting or live:
        while waiting and len(live) < 4:
            name, rid = waiting.pop(0)
            tags[name] = rid
            live[name] = [rid, 0, len(seqs[rid]) <= 2 or rng.random() < 0.3]
        entries, ended = [], []
        for name, st in list(live.items()):
            rid, done, decoding = st
            ids = seqs[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue  # left out of this step, goes on later
            left = len(ids) - done
            if decoding or left == 1:
                n = 1
            else:
                n = min(left, rng.choice([2, 3, 5, 8, 13, 16, 17]))
                if left - n <= 12 and rng.random() < 0.5:
                    st[2] = True  # the rest one token at a time
            entries.append((name, ids[done:done + n], "all"))
            st[1] = done + n
            if st[1] == len(ids):
                ended.append(name)
                del live[name]
        if entries:
            tr.step(entries, end=ended)
    return tr, tags


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def case(request, tmp_path_factory):
    case = dict(CONFIGS[request.param])
    folder = tmp_path_factory.mktemp(request.param)
    plain.write_random_model(folder, case["raw"], case["seed"], dtype=torch.bfloat16)
    sharpen_attention(folder)
    case["folder"] = folder
    case["seqs"] = _sequences(case)
    case["expect"] = plain_logits(folder, case["seqs"])
    case["bf16_noise"] = bfloat16_noise(folder, case["seqs"], case["expect"])
    case["trace"], case["tags"] = _build_trace(case["seqs"])
    return case


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_matches_the_plain_implementation(case, dtype, tmp_path):
    tr, tags = case["trace"], case["tags"]
    # the pool holds exactly what the trace's live requests need at their largest, so the pages
    # of ended requests are handed out again (the trace has far more requests than that)
    got = run_trace(case["folder"], dtype, tr, tmp_path, page_size=case["page"])
    assert len(tags) > 12 and got
    scale = max(e.abs().max().item() for e in case["expect"].values())
    tol = TOL_F32 * max(scale, 1.0)
    errors: dict[str, list[float]] = {}
    whole = {}
    for (name, pos, step), row in got.items():
        rid = tags[name]
        expect = case["expect"][rid][pos]
        err = (row - expect).abs().max().item()
        kind = name.split("-")[0][0]
        errors.setdefault(kind, []).append(err)
        if dtype == "float32":
            assert err <= tol, f"{name} position {pos} (step {step}) is off by {err:.3e} (tolerance {tol:.1e})"
        if kind == "w":
            whole[(rid, pos)] = row
    assert set(errors) == {"w", "d", "c", "m"}
    if dtype == "bfloat16":
        for kind, errs in errors.items():
            check_bfloat16(torch.tensor(errs), case["bf16_noise"], f"cut {kind}")
    # every position of every request was seen whole, and again in the other cuts
    assert len(whole) == sum(len(s) for s in case["seqs"].values())
    if dtype == "float32":
        # the 32-bit kernels sum in an order that does not depend on the cut: bit-equal
        for (name, pos, step), row in got.items():
            assert torch.equal(row, whole[(tags[name], pos)]), f"{name} position {pos} differs from the whole run"


def test_float32_logits_survive_a_larger_pool_and_other_pages(case, tmp_path):
    """Where a request's pages lie must not matter."""
    tr = Trace()
    rid = max(case["seqs"], key=lambda r: len(case["seqs"][r]))
    ids = case["seqs"][rid]
    tr.step([("pad", ids[:19], [])])  # takes the first pages, so the next request starts elsewhere
    tr.step([("x", ids, "all")], end=["x", "pad"])
    got = run_trace(case["folder"], "float32", tr, tmp_path, max_tokens=1024, page_size=case["page"])
    for (name, pos, step), row in got.items():
        assert (row - case["expect"][rid][pos]).abs().max().item() <= TOL_F32
