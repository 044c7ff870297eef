"""Attention with normed, rotated queries and keys, one or two score maps per head, and values of their own size.

Parameters: ``hidden_size, n_heads, n_kv_heads`` (query head h reads key/value head h // (n_heads / n_kv_heads)),
``dim`` (query/key entries of ONE score map), ``vdim`` (value entries per head), ``maps`` (1, or 2 for differential
attention), ``softmax_scale``, ``window`` (0: every earlier position; w: a token sees itself and the w - 1 before
it), ``cache_window`` (what the cache must keep: the largest window of the layers that read it, 0 for all), ``eps``,
``rot`` = {base, dims, scaling?}, ``bias`` (the four projections have biases), ``own_kv`` (false for a layer that
reads the cached keys and values of an earlier layer and has no key/value tensors of its own) and, with two maps,
``diff``.

Per head and map the queries and keys are brought to unit rms over ``dim`` and multiplied by a weight shared by
all heads and maps, then their first ``rot.dims`` entries are rotated (entry i with entry i + dims/2).  With two
maps each map is a softmax attention of its own over the SAME values, and the head's result is
a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number for the layer; that result is
brought to unit rms over its vdim entries (no weight) and multiplied by 1 - diff.  The cache keeps one row per
position: the kv heads' keys (after norm and rotation), then their values.

Switches for other designs, each with its constants: ``qk_norm`` false leaves queries and keys as the projections
give them (no ``q_norm`` / ``k_norm`` tensors); ``rot_layout`` ``"pairs"`` turns entry 2i with entry 2i + 1 instead
of entry i with entry i + dims/2; ``chunk`` c > 0 replaces the window by chunks of c positions counted from the
sequence's position 0 (position p sees p - p % c .. p; the cache keeps everything); ``head_gate`` multiplies head
h's result by sigmoid(G x)_h, one number per head from the mixer's own input (tensor ``gate`` [heads, hidden], no
bias), before the output projection.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, RowCacheSpec, TensorSpec, register_part
from .linear import Linear
from .position import rotary_frequencies


class MappedAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads = int(p("hidden_size")), int(p("n_heads"))
        self.n_kv_heads = int(p("n_kv_heads", self.n_heads))
        self.dim, self.vdim, self.maps = int(p("dim")), int(p("vdim")), int(p("maps", 1))
        self.scale, self.eps = float(p("softmax_scale")), float(p("eps"))
        self.window = int(p("window", 0))
        self.cache_window = int(p("cache_window", self.window))
        self.own_kv = bool(p("own_kv", True))
        self.bias = bool(p("bias", False))
        self.diff = float(p("diff", 0.0))
        self.qk_norm = bool(p("qk_norm", True))
        self.rot_layout = p("rot_layout", "half")
        self.chunk = int(p("chunk", 0))
        self.head_gate = bool(p("head_gate", False))
        if self.rot_layout not in ("half", "pairs"):
            raise ConfigError(f"mapped attention: rot_layout '{self.rot_layout}' is not 'half' or 'pairs'")
        if self.chunk < 0 or (self.chunk and self.window):
            raise ConfigError("mapped attention: chunks of positions and a window exclude one another")
        if self.maps not in (1, 2):
            raise ConfigError(f"mapped attention has one or two score maps, got {self.maps}")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"mapped attention: {self.n_heads} heads do not split over {self.n_kv_heads} kv heads")
        if self.window and self.cache_window and self.cache_window < self.window:
            raise ConfigError("mapped attention: the cache keeps fewer positions than the window sees")
        rot = p("rot")
        self.rot_dims = int(rot["dims"])
        if self.rot_dims > self.dim or self.rot_dims % 2:
            raise ConfigError(f"mapped attention: {self.rot_dims} rotated entries do not fit a map of {self.dim}")
        self.freqs, self.magnitude = rotary_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
        self.q_width = self.n_heads * self.maps * self.dim
        self.k_width = self.n_kv_heads * self.maps * self.dim
        self.v_width = self.n_kv_heads * self.vdim

    def tensor_specs(self):
        D, name = self.hidden_size, self.tensor_name
        specs = [TensorSpec(name("q"), (self.q_width, D))]
        if self.qk_norm:
            specs.append(TensorSpec(name("q_norm"), (self.dim,), role="vector", init="norm_weight"))
        widths = [("q_bias", self.q_width)]
        if self.own_kv:
            specs += [TensorSpec(name("k"), (self.k_width, D)), TensorSpec(name("v"), (self.v_width, D))]
            if self.qk_norm:
                specs.append(TensorSpec(name("k_norm"), (self.dim,), role="vector", init="norm_weight"))
            widths += [("k_bias", self.k_width), ("v_bias", self.v_width)]
        if self.head_gate:
            specs.append(TensorSpec(name("gate"), (self.n_heads, D)))
        specs.append(TensorSpec(name("out"), (D, self.n_heads * self.vdim), init="residual_projection"))
        widths.append(("out_bias", D))
        if self.bias:
            specs += [TensorSpec(name(role), (n,), role="vector", init="bias") for role, n in widths]
        if self.maps == 2:
            specs += [TensorSpec(name(role), (self.dim,), role="vector", init="bias") for role in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def cache_spec(self):
        return RowCacheSpec(self.k_width + self.v_width, self.cache_window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        roles = ["q"] + (["k", "v"] if self.own_kv else [])
        mats = [t(r) for r in roles]
        biases = [t(r + "_bias") for r in roles] if self.bias else None
        self.gate_at = None
        if self.head_gate:
            # the gates ride in the same product, after q | k | v; rows of zeros keep the stacked row a whole
            # number of 16-byte pieces
            self.gate_at = len(mats) + 1
            pad = -(sum(m.shape[0] for m in mats) + self.n_heads) % 8
            mats.append(t("gate"))
            if pad:
                mats.append(torch.zeros((pad, self.hidden_size), dtype=mats[0].dtype, device=mats[0].device))
            if biases is not None:
                biases.append(torch.zeros(self.n_heads + pad, dtype=torch.float32, device=biases[0].device))
        weight = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        bias = torch.cat(biases).contiguous() if biases is not None else None
        self.widths = tuple(m.shape[0] for m in mats)
        self.proj = Linear(weight, bias, runtime)
        self.out = Linear(t("out"), t("out_bias") if self.bias else None, runtime)
        self.q_norm = t("q_norm") if self.qk_norm else None
        self.k_norm = t("k_norm") if self.own_kv and self.qk_norm else None
        self.freq_table = torch.tensor(self.freqs or [0.0], dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.lam, self.out_scale = 0.0, 1.0
        if self.maps == 2:
            # one number for the layer, in float32 like everything around the softmax
            dot = lambda a, b: (t(a).float() * t(b).float()).sum(dtype=torch.float32)
            self.lam = float(torch.exp(dot("lq1", "lk1")) - torch.exp(dot("lq2", "lk2")) + self.diff)
            self.out_scale = 1.0 - self.diff

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T = ctx.n_tokens
        if owns_cache and not self.own_kv:
            raise ConfigError("an attention layer without key and value projections cannot own a cache")
        views = ctx.buffer("mapped.proj" if self.own_kv else "mapped.proj_q", (T, sum(self.widths)), dt, columns=self.widths)
        self.proj(h, out=views[0])
        q = views[1]
        k, v = (views[2], views[3]) if owns_cache else (None, None)
        gate = views[self.gate_at] if self.gate_at is not None else None
        table = ctx.block_tables[cache.group]
        ops.qk_prepare(q, k, v, self.q_norm, self.k_norm, self.freq_table, self.magnitude, self.rot_dims, self.eps,
                       self.n_heads, self.n_kv_heads, self.maps, self.dim, self.vdim, ctx.tok_pos, ctx.tok_seq,
                       table if owns_cache else None, cache.page_tokens, cache.pages if owns_cache else None,
                       pairs=self.rot_layout == "pairs")
        ctx.note("q", q)
        heads = ctx.buffer("mapped.heads", (T, self.n_heads * self.vdim), dt)
        ops.mapped_attention(q, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq, self.n_heads,
                             self.n_kv_heads, self.maps, self.dim, self.vdim, self.scale, self.window, heads,
                             lam=self.lam, out_scale=self.out_scale, eps=self.eps, unit_rms=self.maps == 2,
                             tiles=None if ctx.is_decode else ctx.q_tiles, single_tokens=ctx.is_decode,
                             gate=gate, chunk=self.chunk)
        ctx.note("attn", heads)
        self.out(heads, residual=residual if accumulate else None, out=residual)


register_part("mixer", "mapped_attention", MappedAttention, replace=True)
