"""The engine at the benchmark's own operating points, against the plain implementation: Qwen3-0.6B
and Qwen3-8B layer sizes (fewer layers, random weights), default dispatch, no forced switches.

A 2,048-token prompt in one step and in portions of 1,024 behind the growing prefix; 32 decode steps
at batch 8 replayed from CUDA graphs at a context beyond 2,048; one decode step at batch 40. At these
sizes the steps run through the tcgen05 matrix product and attention (several key splits), the
weight-streaming products, the cluster-merged decode attention and, at batch 40,
the vendor library's products: the test asserts that they did. float32 results must agree bit for
bit between the cuts; bfloat16 results are held to the plain implementation's own bfloat16 noise."""

import random

import pytest
import torch

from miniserve_b200 import ops
from miniserve_b200.cache import CacheManager
from miniserve_b200.config import preset
from miniserve_b200.engine.graphs import DecodeGraphs
from miniserve_b200.engine.loader import load_model
from miniserve_b200.engine.step import StepFunction, StepRow
from miniserve_b200.ops import attention_bf16
from miniserve_b200.sampling import Sampler
from tests.plain import qwen3_plain as plain
from tests.trace_util import check_bfloat16, sharpen_attention

pytestmark = pytest.mark.gpu

PROMPT, DECODE, PAGE = 2048, 32, 16
SIZES = {"0.6b": 3, "8b": 2}  # preset -> layers kept


def _logits_at(cfg, w, ids, places):
    """Plain logits of one whole sequence at some places only (the head over 151,936 words is the
    costly part on the CPU)."""
    h = plain.hidden_states(cfg, w, ids)[torch.tensor(places)]
    return (plain.rms_norm(h, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T).float()


@pytest.fixture(scope="module", params=sorted(SIZES))
def case(request, tmp_path_factory):
    raw = preset(request.param)
    raw["num_hidden_layers"] = SIZES[request.param]
    path = tmp_path_factory.mktemp("op_" + request.param.replace(".", "_"))
    plain.write_random_model(path, raw, seed=11, dtype=torch.bfloat16)
    sharpen_attention(path, 2.0)
    rng = random.Random(3)
    vocab = raw["vocab_size"]
    seq_a = [rng.randrange(vocab) for _ in range(PROMPT + DECODE)]
    seq_b = seq_a[:PROMPT] + [rng.randrange(vocab) for _ in range(DECODE)]  # the same prompt, other decoded tokens
    # 64 places of the prompt: its ends, page and tile edges, and a random sample
    places = sorted({0, 1, 15, 16, 17, 127, 128, 255, 256, 1023, 1024, 1025, PROMPT - 2, PROMPT - 1}
                    | set(rng.sample(range(PROMPT), 50)))
    tail = list(range(PROMPT, PROMPT + DECODE))
    cfg = plain.read_config(path)
    w32, w16 = plain.read_weights(path, torch.float32), plain.read_weights(path, torch.bfloat16)
    expect = {"a": _logits_at(cfg, w32, seq_a, places + tail), "b": _logits_at(cfg, w32, seq_b, tail)}
    rough = {"a": _logits_at(cfg, w16, seq_a, places + tail), "b": _logits_at(cfg, w16, seq_b, tail)}
    errs = torch.cat([(rough[k] - expect[k]).abs().max(dim=1).values for k in expect])
    return dict(path=path, raw=raw, seq_a=seq_a, seq_b=seq_b, places=places, expect=expect,
                noise=(errs.max().item(), errs.mean().item()))


class _Seen:
    """Counts which kernels the steps ran through."""

    def __init__(self, monkeypatch):
        self.tc_gemm = self.tc_attention = self.blas = 0
        self.tc_attention_splits, self.decode_splits = [], []
        from miniserve_b200.ops import blas

        linear_tc, tc_prefill, splits, gemm = ops.linear_tc, ops.attention_tc_prefill, attention_bf16.choose_splits, blas.gemm_bf16
        qkv_tc = ops.qkv_norm_rope_kv

        def count_qkv(*a, **k):  # the q|k|v product with norm, rotation and cache write in its epilogue
            self.tc_gemm += 1
            return qkv_tc(*a, **k)

        def count_tc(*a, **k):
            self.tc_gemm += 1
            return linear_tc(*a, **k)

        def count_attention(out, q, k_pool, v_pool, ctx, group, *a, **k):
            r = tc_prefill(out, q, k_pool, v_pool, ctx, group, *a, **k)
            self.tc_attention += 1
            self.tc_attention_splits += [v[0] for key, v in ctx.step_cache.items() if key[0] == "attn_tc_plan"]
            return r

        def count_splits(*a, **k):
            n = splits(*a, **k)
            self.decode_splits.append(n)
            return n

        def count_blas(*a, **k):
            self.blas += 1
            return gemm(*a, **k)

        monkeypatch.setattr(ops, "linear_tc", count_tc)
        monkeypatch.setattr(ops, "qkv_norm_rope_kv", count_qkv)
        monkeypatch.setattr(ops, "attention_tc_prefill", count_attention)
        monkeypatch.setattr(attention_bf16, "choose_splits", count_splits)
        monkeypatch.setattr(blas, "gemm_bf16", count_blas)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_whole_and_in_portions_then_graph_decode_at_batch_8_and_a_step_at_batch_40(case, dtype, monkeypatch):
    seen = _Seen(monkeypatch)
    seq_a, seq_b, places = case["seq_a"], case["seq_b"], case["places"]
    _, _, model = load_model(case["path"], dtype, "cuda:0")
    vocab = model.spec.vocab_size
    rows_max = 40
    pages = rows_max * (-(-(PROMPT + DECODE + 1) // PAGE)) + 4
    cache = CacheManager(model.entry_caches, pages, PAGE, rows_max, dtype=model.dtype, device=model.device, poison=True)
    step = StepFunction(model, cache)
    prompt = seq_a[:PROMPT]

    # ---- the prompt whole, and in two portions behind the growing prefix
    whole_rc = cache.new_request()
    whole = step.run([StepRow(whole_rc, prompt, places)]).clone()
    first = [p for p in places if p < 1024]
    cut_rc = cache.new_request()
    cut = torch.cat([step.run([StepRow(cut_rc, prompt[:1024], first)]),
                     step.run([StepRow(cut_rc, prompt[1024:], [p - 1024 for p in places if p >= 1024])])])
    step.check_status()
    if dtype == "bfloat16":
        assert seen.tc_gemm >= 2 * len(model.layers), "the prompt steps did not run this package's tcgen05 products"
        assert seen.tc_attention >= 3 * len(model.layers) and max(seen.tc_attention_splits) > 1, \
            f"the tcgen05 attention did not cut the keys of a lone prompt: {seen.tc_attention_splits}"

    # ---- 32 decode steps at batch 8 from CUDA graphs: rows 0 and 7 are checked, the others keep them company
    batch = [whole_rc, cut_rc] + [cache.new_request() for _ in range(6)]
    for i in range(2, 8, 2):  # the other six requests get the same prompt, two per step
        step.run([StepRow(batch[i], prompt, []), StepRow(batch[i + 1], prompt, [])])
    graphs = DecodeGraphs(step, Sampler(model.device, vocab, 8), 8)
    decoded = {0: [], 7: []}
    for t in range(DECODE):
        tokens = [seq_a[PROMPT + t]] + [seq_b[PROMPT + t]] * 7
        got = graphs.run([StepRow(rc, [tok], (0,)) for rc, tok in zip(batch, tokens)], None)
        logits = graphs._graphs[(8, "greedy", 0)].logits
        assert got.tolist() == torch.argmax(logits[:8], -1).tolist()
        for r in decoded:
            decoded[r].append(logits[r].clone())
    step.check_status()
    assert len(graphs._graphs) == 1 and graphs.replayed_launches > 0
    if dtype == "bfloat16":
        assert seen.decode_splits and all(2 <= n <= 8 for n in seen.decode_splits), \
            f"decode attention at batch 8 was not merged inside a cluster: splits {set(seen.decode_splits)}"

    # ---- one decode step at batch 40 (beyond the weight-streaming products): eagerly
    more = [cache.new_request() for _ in range(rows_max - 8)]
    for i in range(0, len(more), 2):
        step.run([StepRow(more[i], prompt, []), StepRow(more[i + 1], prompt, [])])
    for rc in batch:
        cache.release(rc)
    fresh = [cache.new_request() for _ in range(8)]  # their pages are used again at once, by new requests
    for i in range(0, 8, 2):
        step.run([StepRow(fresh[i], prompt, []), StepRow(fresh[i + 1], prompt, [])])
    everyone = fresh + more
    blas_before = seen.blas
    tokens = [seq_a[PROMPT]] + [seq_b[PROMPT]] * (rows_max - 1)
    wide = step.run([StepRow(rc, [tok], (0,)) for rc, tok in zip(everyone, tokens)])
    step.check_status()
    if dtype == "bfloat16":
        assert seen.blas > blas_before, "a decode step of 40 rows did not go to the library's products"
    for rc in everyone:
        cache.release(rc)
    assert cache.is_idle()

    # ---- against the plain implementation
    expect_a, expect_b = case["expect"]["a"], case["expect"]["b"]
    got_a = torch.cat([whole, torch.stack(decoded[0])]).cpu()
    got_b = torch.stack(decoded[7]).cpu()
    results = {"whole + graph decode (row 0)": (got_a, expect_a), "graph decode (row 7)": (got_b, expect_b),
               "in portions": (cut.cpu(), expect_a[:len(places)]),
               "batch 40": (wide[[0, rows_max - 1]].cpu(), torch.stack([expect_a[len(places)], expect_b[0]]))}
    scale = max(1.0, expect_a.abs().max().item())
    for name, (got, want) in results.items():
        err = (got - want).abs().max(dim=1).values
        if dtype == "float32":
            assert err.max().item() <= 1e-4 * scale, f"{name}: place {int(err.argmax())} is off by {err.max().item():.3e}"
        else:
            check_bfloat16(err, case["noise"], name)
    if dtype == "float32":  # however the tokens were cut and batched: the same bits
        assert torch.equal(whole, cut)
        assert torch.equal(wide[0], decoded[0][0]) and torch.equal(wide[rows_max - 1], decoded[7][0])
