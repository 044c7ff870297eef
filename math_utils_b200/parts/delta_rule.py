"""The gated delta rule: a recurrent mixer whose state per head is a matrix S [dim, vdim] that every token first
lets decay, then corrects along its key, then reads with its query.

Parameters: ``hidden_size, n_heads`` (value heads), ``n_kv_heads`` (query/key heads: head h reads
h // (n_heads / n_kv_heads)), ``dim`` (query/key entries), ``vdim`` (value entries), ``conv`` (taps of the short
convolution), ``eps`` (of the output norm).

From the mixer's input x: q = Q x and k = K x (n_kv_heads x dim), v = V x (n_heads x vdim); each channel of q, k, v
passes a causal convolution over time (zeros before a sequence's start, the last tap on the current token, no bias)
and silu; q and k become unit vectors per head, y / sqrt(sum y^2 + 1e-6), and q is multiplied by dim^(-1/2);
beta = sigmoid(B x) and decay = exp(-exp(A_log) softplus(A x + dt_bias)), one each per head.  Per head and token
    S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
o is brought to unit rms over vdim, multiplied by a weight of vdim entries (the same for every head) and by
silu(G x), and goes through the output matrix.  A sequence's state (the convolution's last taps - 1 inputs and every
head's S) is float32 and lives in the sequence's cache slot; gates, decays and the recurrence are float32 whatever
the compute dtype.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, StateCacheSpec, TensorSpec, register_part
from .linear import Linear


class GatedDeltaMixer(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads = int(p("hidden_size")), int(p("n_heads"))
        self.n_kv_heads = int(p("n_kv_heads", self.n_heads))
        self.dim, self.vdim, self.taps = int(p("dim")), int(p("vdim")), int(p("conv"))
        self.eps = float(p("eps"))
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"gated delta mixer: {self.n_heads} heads do not split over {self.n_kv_heads} key heads")
        self.qk_width = self.n_kv_heads * self.dim
        self.inner = self.n_heads * self.vdim
        self.channels = 2 * self.qk_width + self.inner                        # what the convolution sees: q | k | v
        self.tail_values = (self.taps - 1) * self.channels

    def tensor_specs(self):
        name, H, D = self.tensor_name, self.n_heads, self.hidden_size
        return (TensorSpec(name("q"), (self.qk_width, D)), TensorSpec(name("k"), (self.qk_width, D)),
                TensorSpec(name("v"), (self.inner, D)),
                TensorSpec(name("q_conv"), (self.qk_width, self.taps), role="vector", init="conv"),
                TensorSpec(name("k_conv"), (self.qk_width, self.taps), role="vector", init="conv"),
                TensorSpec(name("v_conv"), (self.inner, self.taps), role="vector", init="conv"),
                TensorSpec(name("beta"), (H, D)), TensorSpec(name("decay"), (H, D)),
                TensorSpec(name("A_log"), (H,), role="vector", init="bias"),
                TensorSpec(name("dt_bias"), (H,), role="vector", init="bias"),
                TensorSpec(name("norm"), (self.vdim,), role="vector", init="norm_weight"),
                TensorSpec(name("gate"), (self.inner, D)),
                TensorSpec(name("out"), (D, self.inner), init="residual_projection"))

    def cache_spec(self):
        return StateCacheSpec(self.tail_values + self.inner * self.dim)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        if self.dim > runtime.ops.delta_scan_max_dk():
            raise ConfigError(f"gated delta mixer: keys of {self.dim} entries are more than the scan's "
                              f"{runtime.ops.delta_scan_max_dk()}")
        mats = [t(r) for r in ("q", "k", "v", "gate", "beta", "decay")]
        self.widths = [m.shape[0] for m in mats]
        pad = -sum(self.widths) % 8
        if pad:
            mats.append(torch.zeros((pad, self.hidden_size), dtype=mats[0].dtype, device=mats[0].device))
        self.total = sum(self.widths) + pad
        self.proj = Linear(torch.cat(mats, dim=0).contiguous(), None, runtime)
        self.out = Linear(t("out"), None, runtime)
        self.conv_weight = torch.cat([t("q_conv"), t("k_conv"), t("v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = t("A_log"), t("dt_bias")
        self.norm_weight = t("norm").repeat(self.n_heads).contiguous()       # the same weight for every head

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T, C, inner, H, G = ctx.n_tokens, self.channels, self.inner, self.n_heads, self.n_kv_heads
        if not owns_cache:
            raise ConfigError("a gated delta mixer keeps its own state: it cannot read another layer's")
        u = ctx.buffer("delta.proj", (T, self.total), dt)
        self.proj(h, out=u)
        conv_in, gate = u[:, :C], u[:, C:C + inner]
        b_raw, a_raw = u[:, C + inner:C + inner + H], u[:, C + inner + H:C + inner + 2 * H]
        qkv = ctx.buffer("delta.qkv", (T, C), torch.float32)
        ops.ssd_conv(conv_in, self.conv_weight, None, ctx.tok_seq, ctx.seq_first, ctx.seq_slots, cache.values,
                     ctx.is_decode, qkv)
        kq = ctx.buffer("delta.kq", (T, G), torch.float32)
        beta = ctx.buffer("delta.beta", (T, H), torch.float32)
        decay = ctx.buffer("delta.decay", (T, H), torch.float32)
        ops.delta_prepare(qkv, b_raw, a_raw, self.a_log, self.dt_bias, H, G, self.dim, self.dim ** -0.5, kq, beta, decay)
        o = ctx.buffer("delta.o", (T, inner), torch.float32)
        ops.delta_scan(qkv, kq, beta, decay, H, G, self.dim, self.vdim, ctx.seq_first, ctx.seq_slots, cache.values,
                       self.tail_values, o)
        ctx.note("scan", o)
        gated = ctx.buffer("delta.gated", (T, inner), dt)
        ops.gated_group_norm(o, gate, self.norm_weight, H, self.eps, gated, gate_after=True)
        ctx.note("attn", gated)
        self.out(gated, residual=residual if accumulate else None, out=residual)


register_part("mixer", "gated_delta", GatedDeltaMixer, replace=True)
