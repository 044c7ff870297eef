"""Dense two-matrix feed-forward: up projection, activation, down projection
(include/ai/LocalModel.hpp:3767-3774).  The activation is a parameter:
``gelu_new`` (tanh form, include/ai/LocalModel.hpp:1388-1391), ``gelu``
(erf form) or ``xielu``: with two learned numbers (p, q) in the tensor
``act_params``, softplus(p) z^2 + z / 2 for z > 0 and
(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 below, a launch of its own between
the two products.  Parameter ``bias``: true (both biases must be in the file),
``"if_present"`` or false."""
from __future__ import annotations

from ..config.base import ConfigError, PartSpec
from .base import FeedForward, TensorSpec, register_part
from .linear import Linear

ACTIVATIONS = ("gelu_new", "gelu")
LEARNED_ACTIVATIONS = ("xielu",)


class DenseFeedForward(FeedForward):
    takes_lazy_norm = True
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden_size = int(self.param("hidden_size"))
        self.inner_size = int(self.param("inner_size"))
        self.activation = self.param("activation")
        if self.activation not in ACTIVATIONS + LEARNED_ACTIVATIONS:
            raise ConfigError(f"dense_ffn: activation '{self.activation}' is not one of "
                              f"{', '.join(ACTIVATIONS + LEARNED_ACTIVATIONS)}")
        self.in_out = self.param("weight_layout", "out_in") == "in_out"

    def _matrix(self, role, out_f, in_f, init):
        shape = (in_f, out_f) if self.in_out else (out_f, in_f)
        return TensorSpec(self.tensor_name(role), shape, role="matrix", transpose=self.in_out, init=init)

    def tensor_specs(self):
        d, i = self.hidden_size, self.inner_size
        learned = ((TensorSpec(self.tensor_name("act_params"), (2,), role="vector", init="act_params"),)
                   if self.activation in LEARNED_ACTIVATIONS else ())
        return ((self._matrix("up_weight", i, d, "normal"),) + self.bias_spec("up_bias", i)
                + (self._matrix("down_weight", d, i, "residual_projection"),) + self.bias_spec("down_bias", d) + learned)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.up = Linear(tensors[self.tensor_name("up_weight")], self.bias_tensor(tensors, "up_bias"), runtime)
        self.down = Linear(tensors[self.tensor_name("down_weight")], self.bias_tensor(tensors, "down_bias"), runtime)
        self.act_params = (tensors[self.tensor_name("act_params")].contiguous()
                           if self.activation in LEARNED_ACTIVATIONS else None)

    def forward(self, h, residual, ctx, accumulate: bool = True) -> None:
        hidden = None if ctx is None else ctx.buffer("feed_forward.hidden", (ctx.n_tokens, self.inner_size),
                                                     self.runtime.dtype)
        if self.act_params is not None:
            u = self.runtime.ops.xielu(self.up(h, out=hidden), self.act_params)
        else:
            u = self.up(h, act=self.activation, out=hidden)
        if ctx is not None:
            ctx.note("act", u)
        self.down(u, residual=residual if accumulate else None, out=residual)


class GatedFeedForward(FeedForward):
    """down(act(gate h) * (up h)) with three matrices and no biases; ``activation`` is ``silu``, ``gelu_new`` or
    ``gelu``.  The gate and up matrices are stacked, so one product gives both halves of a row."""
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden_size = int(self.param("hidden_size"))
        self.inner_size = int(self.param("inner_size"))
        self.activation = self.param("activation", "silu")
        if self.activation not in ("silu",) + ACTIVATIONS:
            raise ConfigError(f"gated_ffn: activation '{self.activation}' is not one of silu, {', '.join(ACTIVATIONS)}")

    def tensor_specs(self):
        d, i, name = self.hidden_size, self.inner_size, self.tensor_name
        return (TensorSpec(name("gate_weight"), (i, d)), TensorSpec(name("up_weight"), (i, d)),
                TensorSpec(name("down_weight"), (d, i), init="residual_projection"))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        import torch
        both = torch.cat([tensors[self.tensor_name("gate_weight")], tensors[self.tensor_name("up_weight")]], dim=0)
        self.gate_up = Linear(both.contiguous(), None, runtime)
        self.down = Linear(tensors[self.tensor_name("down_weight")], None, runtime)

    def forward(self, h, residual, ctx, accumulate: bool = True) -> None:
        dt = self.runtime.dtype
        both = ctx.buffer("gated_ffn.both", (ctx.n_tokens, 2 * self.inner_size), dt)
        hidden = ctx.buffer("gated_ffn.hidden", (ctx.n_tokens, self.inner_size), dt)
        self.gate_up(h, out=both)
        self.runtime.ops.gated_act(both, hidden, self.activation)
        ctx.note("act", hidden)
        self.down(hidden, residual=residual if accumulate else None, out=residual)


class NoFeedForward(FeedForward):
    """A layer that ends after its mixer."""
    can_overwrite = True

    def forward(self, h, residual, ctx, accumulate: bool = True) -> None:
        if not accumulate:
            residual.zero_()


register_part("feed_forward", "dense_ffn", DenseFeedForward, replace=True)
register_part("feed_forward", "gated_ffn", GatedFeedForward, replace=True)
register_part("feed_forward", "none", NoFeedForward, replace=True)
