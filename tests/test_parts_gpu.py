"""Each part alone against the plain implementation's function for it, and a toy mixer with
state of its own that is registered, built and stepped without touching the package."""

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.cache.manager import KVEntryView
from miniserve_b200.config import (Architecture, LayerSpec, ModelSpec, PartSpec, RunEntry, register_architecture,
                                   resolve, unregister_architecture)
from miniserve_b200.engine.context import StepContext
from miniserve_b200.engine.step import StepFunction, StepRow
from miniserve_b200.parts import (BuildEnv, DecoderModel, FixedState, Part, ResidualStream, WeightDecl, build_part,
                                  register_part, unregister_part)
from miniserve_b200.parts.block import build_block
from miniserve_b200.weights import random_tensors
from tests.kernel_util import PagedBatch, make_context
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


_ctx = make_context


def _tol(dtype, scale=1.0):
    return dict(atol=1e-5 * scale, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2 * scale, rtol=3e-2)


def _bind_random(part, dtype, seed=0, std=0.2):
    tensors = random_tensors(part.all_weights(), seed, dtype=dtype, std=std, device=DEV)
    part.bind_all(tensors)
    return {k: v.float().cpu() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    env = BuildEnv(dtype, DEV)
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=72, eps=1e-5)), env)
    w = _bind_random(norm, dtype)
    res = torch.randn(11, 72, device=DEV)
    pb = PagedBatch([(0, 11)], 16, 1, 16, dtype)
    out = norm.forward(res, None, _ctx(pb))
    assert torch.allclose(out.float().cpu(), plain.rms_norm(res.cpu(), w["weight"], 1e-5), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    env = BuildEnv(dtype, DEV)
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden=40, intermediate=72)), env)
    w = _bind_random(ffn, dtype)
    x = torch.randn(9, 40, device=DEV).to(dtype)
    pb = PagedBatch([(0, 9)], 16, 1, 16, dtype)
    out = ffn.forward(x, _ctx(pb))
    ref = plain.mlp_block({"model.layers.0.mlp." + k: v for k, v in w.items()}, 0, x.float().cpu())
    assert torch.allclose(out.float().cpu(), ref, **_tol(dtype, 3.0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, page", [(4, 2, 16, 8), (6, 1, 48, 16)])
def test_attention_part_whole_and_in_portions(dtype, heads, kv_heads, d, page):
    hidden, eps, theta, n = 56, 1e-5, 1e4, 29
    env = BuildEnv(dtype, DEV)
    spec = PartSpec("gqa_attention", dict(hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=d, qk_norm=True,
                                          qk_norm_eps=eps, position=PartSpec("rope_neox", dict(head_dim=d, theta=theta))))
    att = build_part("mixer", spec, env)
    w = _bind_random(att, dtype)
    x = torch.randn(n, hidden, device=DEV).to(dtype)
    cfg = dict(heads=heads, kv_heads=kv_heads, head_dim=d, eps=eps, theta=theta)
    ref = plain.attention_block(cfg, {"model.layers.0.self_attn." + k: v for k, v in w.items()}, 0, x.float().cpu(),
                                torch.arange(n))
    # whole
    pb = PagedBatch([(0, n)], page, kv_heads, d, dtype, seed=1)
    out = att.forward(x, _ctx(pb), KVEntryView(0, pb.k_pool, pb.v_pool, page))
    assert pb.status.item() == 0
    assert torch.allclose(out.float().cpu(), ref, **_tol(dtype, 2.0))
    # in two portions over the same pages: the second reads what the first wrote
    full = PagedBatch([(0, n)], page, kv_heads, d, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.v_pool, page)
    pb1 = PagedBatch([(0, 18)], page, kv_heads, d, dtype, share=full)
    o1 = att.forward(x[:18].contiguous(), _ctx(pb1), view)
    pb2 = PagedBatch([(18, n - 18)], page, kv_heads, d, dtype, share=full)
    o2 = att.forward(x[18:].contiguous(), _ctx(pb2), view)
    assert torch.allclose(torch.cat((o1, o2)).float().cpu(), ref, **_tol(dtype, 2.0))


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_embedding_and_head(dtype):
    raw = plain.tiny_config_b()
    _, _, spec = resolve(raw)
    env = BuildEnv(dtype, DEV)
    block = build_block(spec.layers[0], env)
    w = _bind_random(block, dtype, std=0.1)
    n, page = 13, 8
    h0 = torch.randn(n, raw["hidden_size"], device=DEV)
    pb = PagedBatch([(0, n)], page, raw["num_key_value_heads"], raw["head_dim"], dtype)
    stream = block.forward(ResidualStream(h0.clone()), _ctx(pb), KVEntryView(0, pb.k_pool, pb.v_pool, page))
    cfg = dict(heads=6, kv_heads=1, head_dim=32, eps=raw["rms_norm_eps"], theta=raw["rope_theta"])
    ref = plain.decoder_layer(cfg, {"model.layers.0." + k: v for k, v in w.items()}, 0, h0.cpu(), torch.arange(n))
    got = stream.total + stream.pending.float()
    assert torch.allclose(got.cpu(), ref, **_tol(dtype, 3.0))

    emb = build_part("embedding", spec.embedding, env)
    head = build_part("head", spec.head, env)
    we, wh = _bind_random(emb, dtype), _bind_random(head, dtype, seed=1)
    ctx = _ctx(pb)
    ctx.token_ids = torch.randint(0, raw["vocab_size"], (n,), dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ctx).cpu(), we["model.embed_tokens.weight"][ctx.token_ids.long().cpu()])
    x = torch.randn(4, raw["hidden_size"], device=DEV).to(dtype)
    logits = head.forward(x, ctx)
    assert logits.dtype == torch.float32
    assert torch.allclose(logits.cpu(), x.float().cpu() @ wh["lm_head.weight"].T, **_tol(dtype, 2.0))


# ------------------------------------------------------------------ a toy mixer with state of its own
class RunningMeanMixer(Part):
    """y_t = W * mean(x_0 .. x_t): needs the sum so far and the count, per request."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = spec["hidden"]

    def weights(self):
        return {"mix.weight": WeightDecl((self.hidden, self.hidden))}

    def bind(self, tensors):
        self.w = tensors["mix.weight"].float()

    def cache_need(self):
        return FixedState((self.hidden + 1,), torch.float32)

    def forward(self, x, ctx, cache):
        if ctx.decode_only:
            # one token per row: everything on the device, from the step's own tables, so that the pass can be
            # captured in a CUDA graph (padding rows carry the spare slot and need no mask)
            slots = ctx.state_slot.long()
            state = cache.state[slots]
            state = torch.where((ctx.q_start == 0)[:, None], torch.zeros_like(state), state)
            sums, counts = state[:, :-1] + x.float(), state[:, -1:] + 1
            cache.state[slots] = torch.cat((sums, counts), dim=1)
            return ((sums / counts) @ self.w.T).to(x.dtype)
        out = torch.empty_like(x)
        at = 0
        for start, n, slot in zip(ctx.host_q_start, ctx.host_q_len, ctx.host_state_slot):
            state = cache.state[slot]
            if start == 0:
                state.zero_()  # a fresh request (or one that is run again) starts from nothing
            assert int(state[-1].item()) == start, "the state does not belong to this request's past"
            sums = state[:-1] + torch.cumsum(x[at:at + n].float(), 0)
            counts = start + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            out[at:at + n] = ((sums / counts[:, None]) @ self.w.T).to(x.dtype)
            state[:-1] = sums[-1]
            state[-1] = start + n
            at += n
        return out


def _toy_spec(raw):
    hidden = raw["hidden_size"]
    norm = PartSpec("rmsnorm", dict(size=hidden, eps=raw["eps"]))
    block = PartSpec("prenorm", dict(names=dict(mixer="mixer.", feed_forward="ffn.", norm1="ln1.", norm2="ln2.")))
    ffn = PartSpec("swiglu", dict(hidden=hidden, intermediate=raw["inter"]))
    att = PartSpec("gqa_attention", dict(hidden=hidden, heads=4, kv_heads=2, head_dim=16, qk_norm=False,
                                         position=PartSpec("rope_neox", dict(head_dim=16, theta=100.0))))
    toy = PartSpec("running_mean", dict(hidden=hidden))
    layers = tuple(LayerSpec(f"layers.{i}.", block, m, ffn, dict(norm1=norm, norm2=norm))
                   for i, m in enumerate([toy, att]))
    # run order: toy, attention, then the toy layer once more (same weights, state of its own)
    return ModelSpec("ToyStateLM", hidden, raw["vocab"],
                     PartSpec("token_embedding", dict(vocab=raw["vocab"], hidden=hidden, name="embed.weight")),
                     layers, (RunEntry(0), RunEntry(1), RunEntry(0)),
                     PartSpec("rmsnorm", dict(size=hidden, eps=raw["eps"])),
                     PartSpec("linear_head", dict(vocab=raw["vocab"], hidden=hidden, tied=True, name="head.weight",
                                                  tied_to="embed.weight")), final_norm_prefix="final.")


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_mixer_with_state_registers_builds_and_steps(dtype):
    register_part("mixer", "running_mean")(RunningMeanMixer)
    register_architecture(Architecture("ToyStateLM", lambda raw: raw, _toy_spec))
    try:
        raw = dict(architectures=["ToyStateLM"], hidden_size=32, inter=48, vocab=61, eps=1e-5)
        _, _, spec = resolve(raw)
        model = DecoderModel(spec, dtype, DEV)
        assert [type(ec.need).__name__ for ec in model.entry_caches] == ["FixedState", "PagedKV", "FixedState"]
        model.bind(random_tensors(model.weight_decls(), 3, dtype=dtype, std=0.3, device=DEV))
        cache = CacheManager(model.entry_caches, 12, 8, max_requests=2, dtype=dtype, device=DEV)
        assert cache.num_groups == 1 and cache.entry_views[0].state is not cache.entry_views[2].state
        step = StepFunction(model, cache)
        ids = torch.randint(0, 61, (30,)).tolist()
        a = cache.new_request()
        whole = step.run([StepRow(a, ids, range(30))])
        cache.release(a)
        # the same tokens in portions, beside another request, in the slot the first one gave back
        b, c = cache.new_request(), cache.new_request()
        outs, i = [], 0
        for n in (7, 2, 1, 12, 8):
            rows = [StepRow(b, ids[i:i + n], range(n))]
            if i < 20:
                rows.append(StepRow(c, ids[::-1][i:i + n], []))
            outs.append(step.run(rows)[:n])
            i += n
        step.check_status()
        got = torch.cat(outs)
        tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=5e-2, rtol=5e-2)
        assert torch.allclose(got, whole, **tol)
        cache.release(b)
        cache.release(c)
        assert cache.is_idle()
        # decode steps replayed from CUDA graphs over the mixer's state: three requests in a bucket of four
        # (one padding row), token by token after a prompt portion, against the whole-sequence result
        from miniserve_b200.engine.graphs import DecodeGraphs
        from miniserve_b200.sampling import Sampler

        cache3 = CacheManager(model.entry_caches, 24, 8, max_requests=4, dtype=dtype, device=DEV)
        step3 = StepFunction(model, cache3)
        graphs = DecodeGraphs(step3, Sampler(DEV, 61, 4), 4)
        seqs = [ids, ids[::-1], ids[5:] + ids[:5]]
        wholes = []
        for seq in seqs:
            rc = cache3.new_request()
            wholes.append(step3.run([StepRow(rc, seq, range(30))]))
            cache3.release(rc)
        rcs = [cache3.new_request() for _ in seqs]
        step3.run([StepRow(rc, seq[:9], []) for rc, seq in zip(rcs, seqs)])
        for t in range(9, 30):
            graphs.run([StepRow(rc, [seq[t]], (0,)) for rc, seq in zip(rcs, seqs)], None)
            logits = graphs._graphs[(4, "greedy", 0)].logits
            for r in range(3):
                assert torch.allclose(logits[r], wholes[r][t], **tol), f"request {r}, token {t}"
        step3.check_status()
        assert len(graphs._graphs) == 1 and graphs.replayed_launches > 0
        for rc in rcs:
            cache3.release(rc)
        assert cache3.is_idle()
    finally:
        unregister_part("mixer", "running_mean")
        unregister_architecture("ToyStateLM")


# ------------------------------------------------------------------ a toy routed feed-forward and a toy position encoding
class TopOneExperts(Part):
    """y = p_e * W2_e relu(W1_e x) for the expert e with the largest router logit (float32 logits and
    softmax over the experts), token by token."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter, self.experts = spec["hidden"], spec["intermediate"], spec["experts"]
        self.chosen = []  # what the router picked, for the test to look at

    def weights(self):
        w = {"router.weight": WeightDecl((self.experts, self.hidden), precision="float32")}
        for e in range(self.experts):
            w[f"experts.{e}.w1"] = WeightDecl((self.inter, self.hidden))
            w[f"experts.{e}.w2"] = WeightDecl((self.hidden, self.inter))
        return w

    def bind(self, tensors):
        self.router = tensors["router.weight"]
        assert self.router.dtype == torch.float32  # kept in 32-bit whatever the run's dtype
        self.w1 = [tensors[f"experts.{e}.w1"] for e in range(self.experts)]
        self.w2 = [tensors[f"experts.{e}.w2"] for e in range(self.experts)]

    def forward(self, x, ctx):
        from miniserve_b200 import ops

        logits = x.float() @ self.router.T
        prob, expert = torch.softmax(logits, -1).max(-1)
        self.chosen.append(expert.cpu())
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (expert == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(ops.linear(x[rows].contiguous(), self.w1[e], stream=ctx.stream))
                y = ops.linear(h, self.w2[e], stream=ctx.stream)
                out[rows] = (y.float() * prob[rows, None]).to(x.dtype)
        return out


class HalvedPositions(Part):
    """A rotary encoding whose angle is floor(position / 2) * inv_freq: neighbours share an angle.
    The framework's q/k kernel takes it as a table of cos and sin per token."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        d = spec["head_dim"]
        self.rotary_dim = d
        self.inv_freq = (1.0 / (spec["theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(env.device)

    def kernel_table(self):
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx):
        angle = (ctx.positions[:ctx.num_tokens] // 2).float()[:, None] * self.inv_freq[None, :]
        return torch.cat((angle.cos(), angle.sin()), dim=1).contiguous()


def _toy_routed_spec(raw):
    hidden = raw["hidden_size"]
    norm = PartSpec("rmsnorm", dict(size=hidden, eps=raw["eps"]))
    block = PartSpec("prenorm", dict(names=dict(mixer="mixer.", feed_forward="ffn.", norm1="ln1.", norm2="ln2.")))
    dense = PartSpec("swiglu", dict(hidden=hidden, intermediate=raw["inter"]))
    routed = PartSpec("top_one_experts", dict(hidden=hidden, intermediate=raw["inter"], experts=3))

    def attention(position):
        return PartSpec("gqa_attention", dict(hidden=hidden, heads=4, kv_heads=2, head_dim=16, qk_norm=True, qk_norm_eps=raw["eps"],
                                              position=position))

    halved = attention(PartSpec("halved_positions", dict(head_dim=16, theta=50.0)))
    plain_rope = attention(PartSpec("rope_neox", dict(head_dim=16, theta=100.0)))
    layers = (LayerSpec("layers.0.", block, halved, routed, dict(norm1=norm, norm2=norm)),
              LayerSpec("layers.1.", block, plain_rope, dense, dict(norm1=norm, norm2=norm)))
    return ModelSpec("ToyRoutedLM", hidden, raw["vocab"],
                     PartSpec("token_embedding", dict(vocab=raw["vocab"], hidden=hidden, name="embed.weight")),
                     layers, (RunEntry(0), RunEntry(1)),
                     PartSpec("rmsnorm", dict(size=hidden, eps=raw["eps"])),
                     PartSpec("linear_head", dict(vocab=raw["vocab"], hidden=hidden, tied=False, name="head.weight")),
                     final_norm_prefix="final.")


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_routed_feed_forward_and_toy_positions_register_build_and_step(dtype):
    register_part("feed_forward", "top_one_experts")(TopOneExperts)
    register_part("position", "halved_positions")(HalvedPositions)
    register_architecture(Architecture("ToyRoutedLM", lambda raw: raw, _toy_routed_spec))
    try:
        raw = dict(architectures=["ToyRoutedLM"], hidden_size=32, inter=48, vocab=67, eps=1e-5)
        _, _, spec = resolve(raw)
        model = DecoderModel(spec, dtype, DEV)
        tensors = random_tensors(model.weight_decls(), 5, dtype=dtype, std=0.3, device=DEV)
        assert tensors["layers.0.ffn.router.weight"].dtype == torch.float32
        model.bind(tensors)
        cache = CacheManager(model.entry_caches, 12, 8, max_requests=2, dtype=dtype, device=DEV)
        step = StepFunction(model, cache)
        routed = model.layers[0].feed_forward
        ids = torch.randint(0, 67, (30,)).tolist()
        a = cache.new_request()
        whole = step.run([StepRow(a, ids, range(30))])
        cache.release(a)
        picked = routed.chosen[-1]
        assert len(set(picked.tolist())) > 1, "the router sent every token to one expert: the test shows nothing"
        # neighbours share an angle: swapping nothing else, position 2k and 2k+1 rotate alike, so
        # the encoding differs from the framework's own; the cut below must not change a logit
        b, c = cache.new_request(), cache.new_request()
        outs, i = [], 0
        for n in (5, 2, 1, 14, 8):
            rows = [StepRow(b, ids[i:i + n], range(n))]
            if i < 20:
                rows.append(StepRow(c, ids[::-1][i:i + n], []))
            outs.append(step.run(rows)[:n])
            i += n
        step.check_status()
        got = torch.cat(outs)
        tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=6e-2)
        assert torch.allclose(got, whole, **tol)
        cache.release(b)
        cache.release(c)
        assert cache.is_idle()
    finally:
        unregister_part("feed_forward", "top_one_experts")
        unregister_part("position", "halved_positions")
        unregister_architecture("ToyRoutedLM")
