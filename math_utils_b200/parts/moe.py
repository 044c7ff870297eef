"""A feed-forward of routed experts.

Parameters: ``hidden_size, inner_size`` (of one expert), ``n_experts, top``, ``router_scale``,
``score`` (``sigmoid`` | ``softmax``), ``renormalize`` (divide the chosen weights by their sum) and
``correction`` (a per-expert term added to the scores for the CHOICE only).  Tensors: ``router``
[experts, hidden], ``correction`` [experts], and per expert ``gate``, ``up`` [inner, hidden] and ``down``
[hidden, inner] whose names carry ``{e}``.  An expert is down(silu(gate h) * (up h)), without biases.

Switches for other designs, each with its constants: ``expert_form`` ``"relu2"`` makes an expert
down(max(up h, 0)^2) with two matrices (no ``gate`` tensors); ``identity`` n > 0 adds n router outputs after
the experts' that stand for identity experts (their result is the input h itself; the router and the
correction have ``n_experts + identity`` rows); ``renorm_eps`` is added to the chosen scores' sum before the
division; ``shared`` = {``inner_size``, ``gate``: bool} adds an expert of the same form that every token
passes through (tensors ``shared_up``, ``shared_down``, with ``expert_form`` gated also ``shared_gate_proj``),
its result multiplied, with ``gate`` true, by sigmoid(g . h), one number per token (tensor ``shared_gate``
[1, hidden]).

Router logits, scores and weights are float32.  The (token, expert) pairs are grouped by expert on the
device, each expert's products run over its own rows only, and the results are summed per token in the
order of the token's choices: no host round trip, so single-token steps can be replayed from a graph.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import FeedForward, TensorSpec, register_part


class RoutedExperts(FeedForward):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.inner_size = int(p("hidden_size")), int(p("inner_size"))
        self.n_experts, self.top = int(p("n_experts")), int(p("top"))
        self.router_scale = float(p("router_scale", 1.0))
        self.score = p("score", "sigmoid")
        self.renormalize = bool(p("renormalize", False))
        self.has_correction = bool(p("correction", False))
        self.form = p("expert_form", "gated_silu")
        self.identity = int(p("identity", 0))
        self.renorm_eps = float(p("renorm_eps", 0.0))
        shared = p("shared", None)
        self.shared_inner = int(shared["inner_size"]) if shared else 0
        self.shared_gated = bool(shared.get("gate", False)) if shared else False
        self.n_outputs = self.n_experts + self.identity          # what the router chooses among
        if self.form not in ("gated_silu", "relu2"):
            raise ConfigError(f"routed_experts: expert_form '{self.form}' is not gated_silu or relu2")
        if self.identity < 0:
            raise ConfigError("routed_experts: identity counts the identity experts, 0 or more")
        if self.score not in ("sigmoid", "softmax"):
            raise ConfigError(f"routed_experts: score '{self.score}' is not sigmoid or softmax")
        if not 1 <= self.top <= self.n_outputs:
            raise ConfigError(f"routed_experts: top {self.top} of {self.n_outputs} experts")

    def tensor_specs(self):
        D, F, name = self.hidden_size, self.inner_size, self.tensor_name
        specs = [TensorSpec(name("router"), (self.n_outputs, D), role="matrix32")]
        if self.has_correction:
            specs.append(TensorSpec(name("correction"), (self.n_outputs,), role="vector", init="bias"))
        gated = self.form == "gated_silu"
        for e in range(self.n_experts):
            if gated:
                specs.append(TensorSpec(name("gate").format(e=e), (F, D)))
            specs += [TensorSpec(name("up").format(e=e), (F, D)),
                      TensorSpec(name("down").format(e=e), (D, F), init="residual_projection")]
        if self.shared_inner:
            S = self.shared_inner
            if gated:
                specs.append(TensorSpec(name("shared_gate_proj"), (S, D)))
            specs += [TensorSpec(name("shared_up"), (S, D)),
                      TensorSpec(name("shared_down"), (D, S), init="residual_projection")]
            if self.shared_gated:
                specs.append(TensorSpec(name("shared_gate"), (1, D), role="matrix32"))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        name = self.tensor_name
        self.router = tensors[name("router")]
        self.correction = tensors[name("correction")] if self.has_correction else None
        stack = lambda role: torch.stack([tensors[name(role).format(e=e)] for e in range(self.n_experts)]).contiguous()
        gated = self.form == "gated_silu"
        self.w_gate = stack("gate") if gated else None
        self.w_up, self.w_down = stack("up"), stack("down")
        self.tile_rows = runtime.ops.moe_tile_rows()
        self.shared_up = self.shared_down = self.shared_gate = None
        if self.shared_inner:
            from .linear import Linear
            up = tensors[name("shared_up")]
            if gated:
                up = torch.cat([tensors[name("shared_gate_proj")], up], dim=0).contiguous()
            self.shared_up = Linear(up, None, runtime)
            self.shared_down = Linear(tensors[name("shared_down")], None, runtime)
            if self.shared_gated:
                self.shared_gate = tensors[name("shared_gate")].reshape(-1).contiguous()

    fuses_output_norm = True           # forward(..., output_norm=): the norm of the result, added into the stream

    def forward(self, h, residual, ctx, accumulate: bool = True, output_norm=None) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T, top, E = ctx.n_tokens, self.top, self.n_experts
        P = T * top
        gated = self.form == "gated_silu"
        gate_of = ctx.buffer("moe.shared_gate", (T,), torch.float32) if self.shared_gate is not None else None
        # tiles of 64 slots where the tensor cores take the products and an expert has the rows to fill them
        tile_rows = self.tile_rows
        if ops.moe_tc_ok(dt, self.hidden_size, self.inner_size) and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0:
            tile_rows = 64 if P >= 48 * E else 32
        max_tiles = P // tile_rows + E                     # every grouping of P pairs into E experts fits
        index = ctx.buffer("moe.index", (3 * P + 3 * max_tiles + 4,), torch.int32)
        expert_of, slot_of, pair_of = index[:P], index[P:2 * P], index[2 * P:3 * P]
        tile_info, n_tiles = index[3 * P: 3 * P + 3 * max_tiles], index[3 * P + 3 * max_tiles:]
        weight_of = ctx.buffer("moe.weight", (P,), torch.float32)
        ops.moe_route(h, self.router, self.correction, top, self.router_scale, expert_of, weight_of,
                      softmax=self.score == "softmax", renormalize=self.renormalize, renorm_eps=self.renorm_eps,
                      gate_weight=self.shared_gate, gate_out=gate_of)
        ops.moe_group(expert_of, self.n_outputs, slot_of, pair_of, tile_info, n_tiles, tile_rows,
                      n_real=E if self.identity else 0)
        ctx.note("route", weight_of)
        hidden = ctx.buffer("moe.hidden", (P, self.inner_size), dt)
        if gated:
            ops.moe_gemm(h, pair_of, top, self.w_gate, self.w_up, tile_info, n_tiles, max_tiles, hidden, tile_rows=tile_rows)
        else:
            ops.moe_gemm(h, pair_of, top, self.w_up, None, tile_info, n_tiles, max_tiles, hidden, tile_rows=tile_rows,
                         act="relu2")
        ctx.note("act", hidden)
        y = ctx.buffer("moe.out", (P, self.hidden_size), torch.float32)
        ops.moe_gemm(hidden, None, top, self.w_down, None, tile_info, n_tiles, max_tiles, y, tile_rows=tile_rows)
        if self.identity or self.shared_inner:
            # the sum also takes the input rows of identity experts and the shared expert's row, times its gate
            shared = None
            if self.shared_inner:
                S = self.shared_inner
                if gated:
                    both = ctx.buffer("moe.shared_both", (T, 2 * S), dt)
                    act = ctx.buffer("moe.shared_hidden", (T, S), dt)
                    self.shared_up(h, out=both)
                    ops.gated_act(both, act, "silu")
                else:
                    act = self.shared_up(h, act="relu2", out=ctx.buffer("moe.shared_hidden", (T, S), dt))
                shared = self.shared_down(act, out=ctx.buffer("moe.shared_out", (T, self.hidden_size), torch.float32))
            extras = dict(identity_rows=h if self.identity else None, shared=shared, shared_gate=gate_of)
            if output_norm is not None:
                mixed = ctx.buffer("moe.mixed", (T, self.hidden_size), torch.float32)
                ops.moe_combine(y, slot_of, weight_of, top, mixed, **extras)
                output_norm.add_into(mixed, residual)
            else:
                ops.moe_combine(y, slot_of, weight_of, top, residual, add=accumulate, **extras)
            return
        if output_norm is not None:
            # residual += norm(sum of the token's experts); Dynamic Tanh in the same launch as the sum
            from .norm import DynamicTanh
            if type(output_norm) is DynamicTanh:
                ops.moe_combine_tanh(y, slot_of, weight_of, top, output_norm.weight, output_norm.bias, output_norm.alpha,
                                     residual)
            else:
                mixed = ctx.buffer("moe.mixed", (T, self.hidden_size), torch.float32)
                ops.moe_combine(y, slot_of, weight_of, top, mixed)
                output_norm.add_into(mixed, residual)
        elif accumulate:
            mixed = ctx.buffer("moe.mixed", (T, self.hidden_size), torch.float32)
            ops.moe_combine(y, slot_of, weight_of, top, mixed)
            residual += mixed
        else:
            ops.moe_combine(y, slot_of, weight_of, top, residual)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
