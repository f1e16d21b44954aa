"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import PagedKV, Part, WeightDecl, build_part, param, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q/k/v projections (no bias), optional per-head RMSNorm of q and k over head_dim, position
    encoding, causal attention with query head h reading kv head h // (heads / kv_heads), output
    projection (miniserve/model/qwen3.py:110-126; scale d^-0.5 at :133-135).

    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``qk_norm`` (bool),
    ``qk_norm_eps``, ``position`` (a PartSpec of category ``position``), optional ``window``
    (a query sees only the last ``window`` keys), optional ``scale``, and ``kv_source``:
    ``own`` (default) or ``shared`` (the layer has no k/v projections and attends over the
    cache of the run entry named by ``RunEntry.cache_of``)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.kv_heads = param(spec, "kv_heads", int)
        self.head_dim = param(spec, "head_dim", int)
        self.qk_norm = bool(spec.get("qk_norm", False))
        self.qk_norm_eps = float(spec.get("qk_norm_eps", 0.0))
        self.window = spec.get("window")
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.kv_source = spec.get("kv_source", "own")
        if self.kv_source not in ("own", "shared"):
            raise ValueError(f"kv_source must be 'own' or 'shared', got {self.kv_source!r}")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are not a multiple of {self.kv_heads} kv heads")
        if self.window is not None and int(self.window) < 1:
            raise ValueError(f"window must be positive, got {self.window}")
        pos_spec = spec.get("position") or PartSpec("none")
        self.position = build_part("position", pos_spec, env)

    @property
    def owns_cache(self) -> bool:
        return self.kv_source == "own"

    def cache_need(self):
        if not self.owns_cache:
            return None
        return PagedKV(self.kv_heads, self.head_dim, int(self.window) if self.window else None)

    def weights(self):
        d = self.head_dim
        w = {"q_proj.weight": WeightDecl((self.heads * d, self.hidden)),
             "o_proj.weight": WeightDecl((self.hidden, self.heads * d))}
        if self.owns_cache:
            w["k_proj.weight"] = WeightDecl((self.kv_heads * d, self.hidden))
            w["v_proj.weight"] = WeightDecl((self.kv_heads * d, self.hidden))
        if self.qk_norm:
            w["q_norm.weight"] = WeightDecl((d,), init="ones_normal")
            if self.owns_cache:
                w["k_norm.weight"] = WeightDecl((d,), init="ones_normal")
        return w

    def stacks(self):
        # one product makes q, k and v (miniserve/model/fused.py:41-95 joins the same rows)
        return {"qkv_proj.weight": ("q_proj.weight", "k_proj.weight", "v_proj.weight")} if self.owns_cache else {}

    def bind(self, tensors):
        if self.owns_cache:
            self.w_qkv = self.joined(tensors, "qkv_proj.weight", self.stacks()["qkv_proj.weight"])
        else:
            self.w_qkv = tensors["q_proj.weight"].contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        self.w_q_norm = tensors["q_norm.weight"].contiguous() if self.qk_norm else None
        self.w_k_norm = tensors["k_norm.weight"].contiguous() if self.qk_norm and self.owns_cache else None

    def forward(self, x: torch.Tensor, ctx, cache):
        """Returns the mixer's addend to the residual stream: a tensor [T, hidden]."""
        t = x.shape[0]
        dt, dev = self.env.dtype, self.w_qkv.device
        q = ctx.buffer("attn.q", (t, self.heads, self.head_dim), dt, dev)
        inv_freq, rotary_dim = self.position.kernel_table()
        indptr, indices = ctx.page_indptr[cache.group], ctx.page_indices[cache.group]
        if (self.owns_cache
                and ops.qkv_fused_ok(x, self.w_qkv, self.heads, self.kv_heads, self.head_dim, rotary_dim if inv_freq is not None else 0,
                                     cache.k, self.w_q_norm, self.w_k_norm)):
            # prompt steps: norm, rotation and cache write in the product's epilogue
            tiled = None
            if inv_freq is not None:
                table = self.position.step_table(ctx)
                key = ("rope_table_tiled", table.data_ptr())
                tiled = ctx.step_cache.get(key)
                if tiled is None:  # once per step; every layer with the same table shares it
                    tiled = ctx.step_cache[key] = ops.rope_table_tiled(table, stream=ctx.stream)
            ops.qkv_norm_rope_kv(q, cache.k, cache.v, x, self.w_qkv, self.w_q_norm, self.w_k_norm, tiled, self.qk_norm_eps,
                                 ctx.positions, ctx.row_of_token, indptr, indices, cache.page_size, stream=ctx.stream)
        else:
            qkv = ops.linear(x, self.w_qkv, stream=ctx.stream, out=ctx.buffer("attn.qkv", (t, self.w_qkv.shape[0]), dt, dev))
            ops.qk_norm_rope_kv(
                q, cache.k if self.owns_cache else None, cache.v if self.owns_cache else None, qkv,
                self.w_q_norm, self.w_k_norm, inv_freq, rotary_dim, self.qk_norm_eps, ctx.positions,
                ctx.row_of_token, indptr, indices, cache.page_size, ctx.status, stream=ctx.stream,
                cos_sin=self.position.step_table(ctx))
        out = ctx.buffer("attn.out", (t, self.heads, self.head_dim), dt, dev)
        ops.attention(out, q, cache.k, cache.v, ctx, cache.group, self.scale, self.window)
        return ops.linear(out.view(t, self.heads * self.head_dim), self.w_o, stream=ctx.stream,
                          out=ctx.buffer("attn.proj", (t, self.w_o.shape[0]), dt, dev))
