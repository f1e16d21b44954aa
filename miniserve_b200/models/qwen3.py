"""The Qwen3 dense decoder as data: its configuration mapped onto parts.

Pre-norm RMSNorm, grouped-query attention with a per-head RMSNorm on q and k before
rotate-half rotary encoding, no biases, SwiGLU feed-forward, tied or untied head
(miniserve/model/qwen3.py:90-218). Tensor names are the checkpoint's own
(miniserve/model/weights.py:60-91). Registered under the name config.json carries in
``architectures``; the reference itself names its class at every call site.
"""

from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

EMBED_NAME = "model.embed_tokens.weight"
HEAD_NAME = "lm_head.weight"


def qwen3_model_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))
    mixer = PartSpec("gqa_attention", dict(
        hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim, qk_norm=True, qk_norm_eps=cfg.rms_norm_eps,
        position=PartSpec("rope_neox", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta)),
        window=None, kv_source="own"))
    ffn = PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size))
    block = PartSpec("prenorm", dict(names=dict(
        mixer="self_attn.", feed_forward="mlp.", norm1="input_layernorm.", norm2="post_attention_layernorm.")))
    layers = tuple(
        LayerSpec(prefix=f"model.layers.{i}.", block=block, mixer=mixer, feed_forward=ffn,
                  norms=dict(norm1=norm, norm2=norm))
        for i in range(cfg.num_hidden_layers))
    return ModelSpec(
        architecture="Qwen3ForCausalLM",
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab_size, hidden=cfg.hidden_size, name=EMBED_NAME)),
        layers=layers,
        run_order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)),
        final_norm_prefix="model.norm.",
        head=PartSpec("linear_head", dict(vocab=cfg.vocab_size, hidden=cfg.hidden_size,
                                          tied=cfg.tie_word_embeddings, name=HEAD_NAME, tied_to=EMBED_NAME)),
    )


QWEN3 = register_architecture(Architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_model_spec), replace=True)
