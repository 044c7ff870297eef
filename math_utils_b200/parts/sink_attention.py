"""Attention with whole-projection norms, a softmax sink, a temperature and a gate per head, and values that layers share.

Parameters: ``hidden_size, n_heads, n_kv_heads`` (query head h reads key/value head h // (n_heads / n_kv_heads)),
``dim`` (query/key entries per head), ``vdim`` (value entries per head), ``softmax_scale``, ``eps``, ``window``
(0: every earlier position), ``bias`` (the q, k, v projections have biases), and the switches
``value_norm`` (each head's value is brought to unit rms over vdim, no weight, before it is cached),
``sink`` (the softmax's denominator counts one more key whose score is zero and which has no value:
p_j = exp(s_j) / (1 + sum exp(s))), ``head_scale`` (a learned number per head multiplies its scores besides
``softmax_scale``), ``head_gate`` (head h's result is multiplied by sigmoid(G x)_h, one number per head, from the
mixer's own input) and ``value_mix``: ``"source"`` (this layer's cached values are also handed to the later layers of
the step), ``"blend"`` (the layer caches (1 - lambda) v + lambda v_source, v_source the source layer's values of the
same token, lambda a learned scalar) or ``"none"``.

The queries, and the keys, are brought to unit rms over ALL their entries at once (every head together) and
multiplied by a weight of that size; there is no rotation.  The cache keeps one row per position: the kv heads'
normed keys, then their values as they are attended to.  Norms, the blend, scores, softmax and the gate are
float32 whatever the compute dtype.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, RowCacheSpec, TensorSpec, register_part
from .linear import Linear

VALUE_MIX = ("none", "source", "blend")


class SinkAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads = int(p("hidden_size")), int(p("n_heads"))
        self.n_kv_heads = int(p("n_kv_heads", self.n_heads))
        self.dim, self.vdim = int(p("dim")), int(p("vdim"))
        self.scale, self.eps = float(p("softmax_scale")), float(p("eps"))
        self.window = int(p("window", 0))
        self.bias = bool(p("bias", False))
        self.value_norm, self.sink = bool(p("value_norm", False)), bool(p("sink", False))
        self.head_scale, self.head_gate = bool(p("head_scale", False)), bool(p("head_gate", False))
        self.value_mix = p("value_mix", "none")
        if self.value_mix not in VALUE_MIX:
            raise ConfigError(f"sink attention: value_mix '{self.value_mix}' is not one of {', '.join(VALUE_MIX)}")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"sink attention: {self.n_heads} heads do not split over {self.n_kv_heads} kv heads")
        self.q_width = self.n_heads * self.dim
        self.k_width = self.n_kv_heads * self.dim
        self.v_width = self.n_kv_heads * self.vdim

    def tensor_specs(self):
        D, name = self.hidden_size, self.tensor_name
        specs = [TensorSpec(name("q"), (self.q_width, D)), TensorSpec(name("k"), (self.k_width, D)),
                 TensorSpec(name("v"), (self.v_width, D)),
                 TensorSpec(name("q_norm"), (self.q_width,), role="vector", init="norm_weight"),
                 TensorSpec(name("k_norm"), (self.k_width,), role="vector", init="norm_weight"),
                 TensorSpec(name("out"), (D, self.n_heads * self.vdim), init="residual_projection")]
        if self.bias:
            specs += [TensorSpec(name(r + "_bias"), (n,), role="vector", init="bias")
                      for r, n in (("q", self.q_width), ("k", self.k_width), ("v", self.v_width))]
        if self.head_scale:
            specs.append(TensorSpec(name("head_scale"), (self.n_heads,), role="vector", init="head_scale"))
        if self.head_gate:
            specs.append(TensorSpec(name("gate"), (self.n_heads, D)))
        if "mix" in self.spec.tensors:
            # a source layer may carry the scalar without using it; a layer that mixes nothing may lack it
            specs.append(TensorSpec(name("mix"), (), role="vector", init="mix", optional=self.value_mix == "none"))
        return specs

    def cache_spec(self):
        return RowCacheSpec(self.k_width + self.v_width, self.window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        roles = ["q", "k", "v"] + (["gate"] if self.head_gate else [])
        mats = [t(r) for r in roles]
        widths = [m.shape[0] for m in mats]
        pad = -sum(widths) % 8                      # rows of the stacked output start on 16-byte boundaries
        if pad:
            mats.append(torch.zeros((pad, self.hidden_size), dtype=mats[0].dtype, device=mats[0].device))
        bias = None
        if self.bias:
            parts = [t(r + "_bias") for r in ("q", "k", "v")]
            rest = sum(widths[3:]) + pad
            if rest:
                parts.append(torch.zeros(rest, dtype=torch.float32, device=parts[0].device))
            bias = torch.cat(parts).contiguous()
        self.widths = tuple(widths) + ((pad,) if pad else ())
        self.proj = Linear(torch.cat(mats, dim=0).contiguous(), bias, runtime)
        self.out = Linear(t("out"), None, runtime)
        self.q_norm, self.k_norm = t("q_norm"), t("k_norm")
        self.head_scales = t("head_scale").contiguous() if self.head_scale else None
        self.mix = float(t("mix")) if self.value_mix == "blend" else 0.0

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T = ctx.n_tokens
        if not owns_cache:
            raise ConfigError("a sink attention layer keeps its own keys and values")
        views = ctx.buffer("sink_attention.proj", (T, sum(self.widths)), dt, columns=self.widths)
        self.proj(h, out=views[0])
        q, k, v = views[1], views[2], views[3]
        gate = views[4] if self.head_gate else None
        first, mode = None, 0
        if self.value_mix != "none":
            first = ctx.buffer("sink_attention.shared_values", (T, self.v_width), torch.float32)
            mode = 1 if self.value_mix == "source" else 2
        table = ctx.block_tables[cache.group]
        ops.qkv_norm_rows(q, k, v, self.q_norm, self.k_norm, self.eps, self.n_kv_heads, self.vdim, self.value_norm,
                          ctx.tok_pos, ctx.tok_seq, table, cache.page_tokens, cache.pages, first, mode, self.mix)
        ctx.note("q", q)
        heads = ctx.buffer("sink_attention.heads", (T, self.n_heads * self.vdim), dt)
        ops.mapped_attention(q, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq, self.n_heads,
                             self.n_kv_heads, 1, self.dim, self.vdim, self.scale, self.window, heads,
                             tiles=None if ctx.is_decode else ctx.q_tiles, single_tokens=ctx.is_decode,
                             head_scale=self.head_scales, sink=self.sink, gate=gate)
        ctx.note("attn", heads)
        self.out(heads, residual=residual if accumulate else None, out=residual)


register_part("mixer", "sink_attention", SinkAttention, replace=True)
