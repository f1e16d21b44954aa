"""Plain, slow restatement of the Qwen3 dense decoder, used only as the tests' oracle.

Whole sequences, no cache, no batching, one function per part, nothing imported from
the product package. Every function cites the place in samplecatalina/mini-serve whose
formula it restates (paths are relative to that project). All arithmetic runs in the
dtype of the weights it is given except where the reference itself goes to float32
(norm statistics, rotation angles); softmax is done in float32 explicitly.

The outputs of this file were compared once with mini-serve's own model code on the
CPU (see ``tests/golden/make_golden.py`` and the ``.json``/``.safetensors`` files
beside it); the tests re-check those stored outputs without needing the reference.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- config

def read_config(model_dir) -> dict:
    """config.json keys as the reference reads them (miniserve/model/qwen3.py:38-55)."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    if raw.get("rope_scaling"):
        raise NotImplementedError("rope_scaling")
    if raw.get("hidden_act", "silu") != "silu":
        raise NotImplementedError("hidden_act")
    return dict(
        hidden=raw["hidden_size"],
        inter=raw["intermediate_size"],
        vocab=raw["vocab_size"],
        layers=raw["num_hidden_layers"],
        heads=raw["num_attention_heads"],
        kv_heads=raw["num_key_value_heads"],
        head_dim=raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"],
        eps=raw["rms_norm_eps"],
        theta=float(raw["rope_theta"]),
        tied=raw.get("tie_word_embeddings", False),
    )


def read_weights(model_dir, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Every tensor of every safetensors file, cast to ``dtype``
    (miniserve/model/weights.py:105-114); tied head aliases the embedding (:135-136)."""
    from safetensors.torch import load_file

    out: dict[str, torch.Tensor] = {}
    for f in sorted(Path(model_dir).glob("*.safetensors")):
        for k, v in load_file(str(f)).items():
            out[k] = v.to(dtype)
    cfg = read_config(model_dir)
    if cfg["tied"]:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out


# --------------------------------------------------------------------------- parts

def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Normalise in float32, cast back, then scale by ``w`` in the input dtype
    (miniserve/model/qwen3.py:78-82)."""
    xf = x.to(torch.float32)
    var = (xf * xf).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return w * xf.to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq[j] = 1/theta^(2j/d) in float32 from an int64 arange; angles = pos*inv_freq
    in float32; cos/sin of [angles, angles] cast to the model dtype
    (miniserve/model/qwen3.py:98-108)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    ang = torch.cat((ang, ang), dim=-1)
    # The cosine and sine of the float32 angle are taken by numpy in float64 and rounded to float32:
    # the value an exact float32 cosine gives. torch's own float32 cosine on the CPU is within an
    # ulp of it almost always, but its first call in a process was seen to return values off by
    # 1.5e-4 at angles of tens of radians (about one process in fifty, on two machines), which
    # moves logits by a thousand times the float32 tolerance of the tests.
    import numpy as np

    wide = ang.to(torch.float64).numpy()
    cos = torch.from_numpy(np.cos(wide)).to(torch.float32)
    sin = torch.from_numpy(np.sin(wide)).to(torch.float32)
    return cos.to(dtype), sin.to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[d/2:], x[:d/2]) (miniserve/model/qwen3.py:85-87)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin, cos/sin broadcast over heads
    (miniserve/model/qwen3.py:121-123). ``x``: [T, heads, d]."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """softmax(q k^T * d^-0.5 + causal mask) v with grouped heads: query head h reads
    key/value head h // (heads / kv_heads) (miniserve/model/attention.py:60-67,
    miniserve/model/qwen3.py:133-135). q: [T, heads, d]; k, v: [T, kv_heads, d].
    Scores and softmax in float32. ``window``: if given, a query at position p sees
    keys p-window+1 .. p only (not used by Qwen3; kernels are tested with it)."""
    t, heads, d = q.shape
    group = heads // k.shape[1]
    scale = d ** -0.5
    out = torch.empty_like(q)
    idx = torch.arange(t)
    allowed = idx[None, :] <= idx[:, None]
    if window is not None:
        allowed &= idx[None, :] > idx[:, None] - window
    for h in range(heads):
        kh, vh = k[:, h // group].float(), v[:, h // group].float()
        s = (q[:, h].float() @ kh.T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = (p @ vh).to(q.dtype)
    return out


def attention_block(cfg: dict, w: dict, i: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """q/k/v projections, per-head RMSNorm of q and k over head_dim with the model's eps,
    rotation, attention, output projection (miniserve/model/qwen3.py:110-126)."""
    p = f"model.layers.{i}.self_attn."
    t = x.shape[0]
    q = (x @ w[p + "q_proj.weight"].T).view(t, cfg["heads"], cfg["head_dim"])
    k = (x @ w[p + "k_proj.weight"].T).view(t, cfg["kv_heads"], cfg["head_dim"])
    v = (x @ w[p + "v_proj.weight"].T).view(t, cfg["kv_heads"], cfg["head_dim"])
    q = rms_norm(q, w[p + "q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[p + "k_norm.weight"], cfg["eps"])
    cos, sin = rope_cos_sin(positions, cfg["head_dim"], cfg["theta"], x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    windows = cfg.get("windows")  # not a Qwen3 key: tests of windowed layers add a window (or None) per layer
    o = causal_attention(q, k, v, window=windows[i] if windows else None)
    return o.reshape(t, cfg["heads"] * cfg["head_dim"]) @ w[p + "o_proj.weight"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    """x * sigmoid(x), what F.silu computes (miniserve/model/qwen3.py:130)."""
    return x * torch.sigmoid(x)


def mlp_block(w: dict, i: int, x: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), no biases (miniserve/model/qwen3.py:128-131)."""
    p = f"model.layers.{i}.mlp."
    g = silu(x @ w[p + "gate_proj.weight"].T)
    return (g * (x @ w[p + "up_proj.weight"].T)) @ w[p + "down_proj.weight"].T


def decoder_layer(cfg: dict, w: dict, i: int, h: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Pre-norm block: h += attn(norm(h)); h += mlp(norm(h)) (miniserve/model/qwen3.py:212-216)."""
    p = f"model.layers.{i}."
    h = h + attention_block(cfg, w, i, rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"]), positions)
    h = h + mlp_block(w, i, rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]))
    return h


def hidden_states(cfg: dict, w: dict, ids: list[int]) -> torch.Tensor:
    """Embedding then every layer, for one whole sequence from position 0
    (miniserve/model/qwen3.py:197-218). Returns [T, hidden] before the last norm."""
    positions = torch.arange(len(ids))
    h = w["model.embed_tokens.weight"][torch.tensor(ids, dtype=torch.long)]
    for i in range(cfg["layers"]):
        h = decoder_layer(cfg, w, i, h, positions)
    return h


def all_logits(cfg: dict, w: dict, ids: list[int]) -> torch.Tensor:
    """Logits at every position of one whole sequence: final norm, then the head
    (miniserve/model/qwen3.py:150-153,183-186). [T, vocab] in the weights' dtype."""
    h = rms_norm(hidden_states(cfg, w, ids), w["model.norm.weight"], cfg["eps"])
    return h @ w["lm_head.weight"].T


# --------------------------------------------------------------------------- sampling

_M32 = 0xFFFFFFFF


def _mix32(x: int) -> int:
    """xor-shift-multiply hash on 32-bit values (miniserve/engine/sampler.py:34-38)."""
    x = (((x >> 16) ^ x) * 0x45D9F3B) & _M32
    x = (((x >> 16) ^ x) * 0x45D9F3B) & _M32
    return (x >> 16) ^ x


def uniform_noise(seed: int, counter: int, vocab: int) -> torch.Tensor:
    """u[v] = ((mix32((key + v*0x9E3779B9) mod 2^32) >> 8) + 0.5) / 2^24 with
    key = mix32(seed ^ mix32(counter)) (miniserve/engine/sampler.py:41-46). Python ints."""
    key = _mix32(seed ^ _mix32(counter))
    vals = [((_mix32((key + v * 0x9E3779B9) & _M32) >> 8) + 0.5) / float(1 << 24) for v in range(vocab)]
    return torch.tensor(vals, dtype=torch.float32)


def sample_token(logits: torch.Tensor, temperature: float, seed: int, counter: int, top_p: float = 1.0) -> int:
    """temperature 0: first maximal index. Else argmax(logits/T + g), g = -log(-log u),
    after masking tokens outside the nucleus (miniserve/engine/sampler.py:86-112)."""
    if temperature == 0:
        return int(torch.argmax(logits))
    z = logits.float() / temperature
    if top_p < 1:
        probs = torch.softmax(z, dim=-1)
        sp, order = torch.sort(probs, descending=True, stable=True)
        before = torch.cumsum(sp, dim=-1) - sp
        keep = torch.empty_like(before, dtype=torch.bool)
        keep[order] = before < top_p
        z = z.masked_fill(~keep, float("-inf"))
    u = uniform_noise(seed, counter, z.shape[-1])
    g = -torch.log(-torch.log(u))
    return int(torch.argmax(z + g))


def generate(cfg: dict, w: dict, prompt: list[int], max_new_tokens: int, temperature: float = 0.0,
             seed: int = 0, stop: frozenset[int] = frozenset(), top_p: float = 1.0) -> list[int]:
    """Recompute the whole sequence for every new token (no cache); the token sampled at
    index ``len(sequence)`` uses that index as the noise counter
    (miniserve/engine/sampler.py:73-76, miniserve/engine/request.py:151-155)."""
    seq, out = list(prompt), []
    for _ in range(max_new_tokens):
        logits = all_logits(cfg, w, seq)[-1]
        tok = sample_token(logits, temperature, seed, len(seq), top_p)
        out.append(tok)
        seq.append(tok)
        if tok in stop:
            break
    return out


# --------------------------------------------------------------------------- random model folders

def tiny_config_a() -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, vocab_size=256,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                max_position_embeddings=128, hidden_act="silu")


def tiny_config_b() -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=224, vocab_size=503,
                num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
                rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                max_position_embeddings=256, hidden_act="silu")


def expected_shapes(raw: dict) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a Qwen3 dense checkpoint (miniserve/model/weights.py:60-91)."""
    h, inter, vocab = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    nq, nkv = raw["num_attention_heads"], raw["num_key_value_heads"]
    d = raw.get("head_dim") or h // nq
    s: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (vocab, h), "model.norm.weight": (h,)}
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (h,)
        s[p + "post_attention_layernorm.weight"] = (h,)
        s[p + "self_attn.q_proj.weight"] = (nq * d, h)
        s[p + "self_attn.k_proj.weight"] = (nkv * d, h)
        s[p + "self_attn.v_proj.weight"] = (nkv * d, h)
        s[p + "self_attn.o_proj.weight"] = (h, nq * d)
        s[p + "self_attn.q_norm.weight"] = (d,)
        s[p + "self_attn.k_norm.weight"] = (d,)
        s[p + "mlp.gate_proj.weight"] = (inter, h)
        s[p + "mlp.up_proj.weight"] = (inter, h)
        s[p + "mlp.down_proj.weight"] = (h, inter)
    if not raw.get("tie_word_embeddings", False):
        s["lm_head.weight"] = (vocab, h)
    return s


def write_random_model(folder, raw: dict, seed: int, std: float = 0.02, dtype=torch.float32) -> None:
    """A model folder with matrices N(0, std) and norm weights 1 + N(0, 0.1), written by the
    tests' own generator (independent of the product's random-weights mode)."""
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, shape in expected_shapes(raw).items():
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        tensors[name] = ((1.0 + 0.1 * t) if len(shape) == 1 else std * t).to(dtype).contiguous()
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    save_file(tensors, str(folder / "model.safetensors"))
