"""Named config.json contents for the random-weights mode and the benchmark.

The reference names models by size and pins checkpoints to download
(miniserve/model/weights.py:24-39); there is no network here, so a preset is just the
config.json of that size. These are data for ``--random PRESET``; no kernel or part
reads a size from this file.
"""

from __future__ import annotations


def _qwen3(hidden, inter, vocab, layers, heads, kv_heads, head_dim, theta, eps, tied, max_pos) -> dict:
    return dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
        hidden_size=hidden, intermediate_size=inter, vocab_size=vocab, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
        rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tied, max_position_embeddings=max_pos,
    )


PRESETS: dict[str, dict] = {
    "tiny-a": _qwen3(64, 128, 256, 2, 4, 2, 16, 10000.0, 1e-6, True, 128),
    "tiny-b": _qwen3(96, 224, 503, 3, 6, 1, 32, 1000000.0, 1e-5, False, 256),
    "0.6b": _qwen3(1024, 3072, 151936, 28, 16, 8, 128, 1000000.0, 1e-6, True, 40960),
    "1.7b": _qwen3(2048, 6144, 151936, 28, 16, 8, 128, 1000000.0, 1e-6, True, 40960),
    "8b": _qwen3(4096, 12288, 151936, 36, 32, 8, 128, 1000000.0, 1e-6, False, 40960),
    "32b": _qwen3(5120, 25600, 151936, 64, 64, 8, 128, 1000000.0, 1e-6, False, 40960),
}


def preset(name: str) -> dict:
    try:
        return dict(PRESETS[name.lower()])
    except KeyError:
        raise ValueError(f"unknown preset {name!r}; expected one of {sorted(PRESETS)}") from None
