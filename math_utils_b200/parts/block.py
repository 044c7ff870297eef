"""Arrangements: how a layer's parts sit around the residual stream.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(include/ai/LocalModel.hpp:3705-3782).  The residual stream stays float32;
mixer and feed-forward add into it in their last product's epilogue.

A prompt step of a layer whose parts are this package's own LayerNorm, causal
attention and two-matrix feed-forward, in bfloat16 at the sizes the tcgen05
kernels take, goes to the library as ONE call that issues the layer's eight
launches (``ops.prompt_layer``): the same kernels through the same entry
points, without the host spending longer on the calls than the device on the
kernels.  Every other layer, step and precision goes part by part.

``sandwich_norm``: x += norm1b(mixer(norm1(x))); x += norm2b(feed_forward(norm2(x))), the two
output norms given as the layer's extra parts ``norm1b`` and ``norm2b``.  A sublayer writes its
result to a float32 buffer, and the output norm adds its normed rows into the residual stream.  A
layer without a feed-forward (kind ``none``) stops after the mixer.

``scaled_pre_norm``: x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x)) with one multiplier m
(parameter ``residual_mult``) on what the sublayers add.  A sublayer writes its result to a float32
buffer; the addition to the stream is made by the launch of the NEXT norm (``ops.residual_add_norm``:
x += m * y, then the normed row), also across layers (``StepContext.pending_join``), so the stream is
read and written once per sublayer.

``parallel_pre_norm``: x += mixer(norm1(x)) + feed_forward(norm2(x)), both sublayers reading the SAME x through a
norm of their own.  Both norms are made before either sublayer adds into the stream (two RMS norms with one eps
by one launch: one pass over x, one statistic, two weights); then the mixer and the feed-forward add into the
float32 stream in their last launches.  A layer without a feed-forward is x += mixer(norm1(x)).
"""
from __future__ import annotations

import torch

from .attention import CausalSelfAttention
from .base import Arrangement, PositionEncoding, register_part
from .feedforward import DenseFeedForward, NoFeedForward
from .norm import IdentityNorm, LayerNorm, RmsNorm


class PreNormBlock(Arrangement):
    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        if ctx.trace is None and not ctx.is_decode and self._whole_layer(x, layer, ctx, cache, owns_cache):
            return
        h = layer.norm1.lazy(x) if layer.mixer.takes_lazy_norm else layer.norm1.forward(x)
        ctx.note("ln1", h)
        layer.mixer.forward(h, x, ctx, cache, owns_cache)
        ctx.note("res1", x)
        h = layer.norm2.lazy(x) if layer.feed_forward.takes_lazy_norm else layer.norm2.forward(x)
        ctx.note("ln2", h)
        layer.feed_forward.forward(h, x, ctx)
        ctx.note("res2", x)

    # ------------------------------------------------------------ the layer as one call
    def _whole_layer(self, x, layer, ctx, cache, owns_cache: bool) -> bool:
        """Runs the layer through ``ops.prompt_layer`` if it is the kind that call is for; False if not."""
        args = getattr(layer, "_prompt_args", None)
        if args is None:
            args = layer._prompt_args = self._layer_args(layer)
        if args is False:
            return False
        mixer, ff = layer.mixer, layer.feed_forward
        rt = mixer.runtime
        ops = rt.ops
        n = ctx.n_tokens
        if (n <= 64 or ctx.q_tiles_wide is None or cache is None or cache.page_tokens != 64
                or type(ctx.position).rotate is not PositionEncoding.rotate
                or x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != mixer.hidden_size):
            return False
        width = mixer.q_width + 2 * mixer.kv_width
        qkv = ctx.buffer("attention.qkv", (n, width), rt.dtype, columns=(mixer.q_width, mixer.kv_width, mixer.kv_width))[0]
        attn = ctx.buffer("attention.out", (n, mixer.q_width), rt.dtype)
        inner = ctx.buffer("feed_forward.hidden", (n, ff.inner_size), rt.dtype)
        normed = ops.scratch("layernorm_out", x.device, n * mixer.hidden_size, torch.bfloat16)
        table = ctx.block_tables[cache.group]
        args.x, args.normed, args.qkv, args.attn, args.inner_buf = (x.data_ptr(), normed.data_ptr(), qkv.data_ptr(),
                                                                    attn.data_ptr(), inner.data_ptr())
        args.tok_pos, args.tok_seq, args.block_table = ctx.tok_pos.data_ptr(), ctx.tok_seq.data_ptr(), table.data_ptr()
        args.tiles_wide, args.tiles = ctx.q_tiles_wide.data_ptr(), ctx.q_tiles.data_ptr()
        args.n_tiles_wide, args.n_tiles = ctx.q_tiles_wide.shape[0], ctx.q_tiles.shape[0]
        args.status = ops.status_word(x.device).data_ptr()
        args.kv_pages, args.n_cache_pages = cache.pages.data_ptr(), cache.pages.shape[0]
        args.max_pages, args.page_tokens = table.shape[1], cache.page_tokens
        args.n_tokens, args.owns_cache = n, int(owns_cache)
        ops.prompt_layer(args)
        return True

    @staticmethod
    def _layer_args(layer):
        """The part of the call's arguments that never changes (weights, sizes), or False for a layer
        that is not made of this package's LayerNorm, causal attention and two-matrix feed-forward in
        bfloat16 at sizes the tcgen05 kernels take."""
        n1, mixer, n2, ff = layer.norm1, layer.mixer, layer.norm2, layer.feed_forward
        if not (type(n1) is LayerNorm and type(n2) is LayerNorm and type(mixer) is CausalSelfAttention
                and type(ff) is DenseFeedForward):
            return False
        rt = mixer.runtime
        if rt.dtype != torch.bfloat16 or not rt.ops.PREFILL_TC or mixer.head_dim != 64:
            return False
        weights = (mixer.qkv.weight, mixer.out.weight, ff.up.weight, ff.down.weight)
        if any(w.dtype != torch.bfloat16 or w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16 or w.shape[1] % 8
               for w in weights):
            return False
        if (mixer.q_width + 2 * mixer.kv_width) % 8 or mixer.q_width % 8 or ff.inner_size % 8 or mixer.hidden_size % 8:
            return False
        ops = rt.ops
        a = ops.PromptLayerArgs()
        ptr = lambda t: None if t is None else t.data_ptr()
        a.ln1_gamma, a.ln1_beta, a.eps1 = ptr(n1.weight), ptr(n1.bias), n1.eps
        a.ln2_gamma, a.ln2_beta, a.eps2 = ptr(n2.weight), ptr(n2.bias), n2.eps
        a.qkv_weight, a.qkv_bias, a.ld_qkv_weight = ptr(mixer.qkv.weight), ptr(mixer.qkv.bias), mixer.qkv.weight.stride(0)
        a.out_weight, a.out_bias, a.ld_out_weight = ptr(mixer.out.weight), ptr(mixer.out.bias), mixer.out.weight.stride(0)
        a.up_weight, a.up_bias, a.ld_up_weight = ptr(ff.up.weight), ptr(ff.up.bias), ff.up.weight.stride(0)
        a.down_weight, a.down_bias, a.ld_down_weight = ptr(ff.down.weight), ptr(ff.down.bias), ff.down.weight.stride(0)
        a.hidden, a.inner, a.act = mixer.hidden_size, ff.inner_size, ops.ACT_CODES[ff.activation]
        a.n_heads, a.n_kv_heads, a.head_dim = mixer.n_heads, mixer.n_kv_heads, mixer.head_dim
        a.scale, a.window = mixer.scale, mixer.window
        return a


class SandwichNormBlock(Arrangement):
    """Where a sublayer reads the stream itself (its input norm is the identity) in bfloat16, the output norm
    before it hands the stream on in bfloat16 from the launch that added to it (``RmsNorm.add_into(copy=)``), so
    the stream is not read again just to be rounded; ``ctx.stream_copy`` is that copy while it is current."""

    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        y = ctx.buffer("sublayer.out", tuple(x.shape), torch.float32)
        h = self._input(layer.norm1, x, ctx)
        ctx.note("ln1", h)
        pair = getattr(layer.mixer, "forward_pair", None)
        if pair is not None and isinstance(layer.extra["norm1b"], RmsNorm):
            # two mixers side by side: their weighted sum is made by the norm's launch as it reads them
            first, second = pair(h, ctx, cache, owns_cache)
            a, b = layer.mixer.scales
            self._join(layer.extra["norm1b"], first, x, ctx, second=(a, second, b))
        else:
            self._sublayer(layer.mixer, y, h, y, ctx, cache, owns_cache)
            self._join(layer.extra["norm1b"], y, x, ctx)
        ctx.note("res1", x)
        if not isinstance(layer.feed_forward, NoFeedForward):
            h = self._input(layer.norm2, x, ctx)
            ctx.note("ln2", h)
            if getattr(layer.feed_forward, "fuses_output_norm", False):
                layer.feed_forward.forward(h, x, ctx, output_norm=layer.extra["norm2b"])
                ctx.stream_copy = None
            else:
                self._sublayer(layer.feed_forward, y, h, y, ctx)
                self._join(layer.extra["norm2b"], y, x, ctx)
        ctx.note("res2", x)

    @staticmethod
    def _input(norm, x, ctx):
        if isinstance(norm, IdentityNorm) and ctx.stream_copy is not None:
            return ctx.stream_copy
        return norm.forward(x)

    @staticmethod
    def _join(norm, y, x, ctx, second=None) -> None:
        ctx.stream_copy = None
        if isinstance(norm, RmsNorm):
            copy = ctx.buffer("stream.copy", tuple(x.shape), torch.bfloat16) if norm.runtime.dtype == torch.bfloat16 else None
            norm.add_into(y, x, copy=copy, second=second)
            ctx.stream_copy = copy
        else:
            norm.add_into(y, x)

    @staticmethod
    def _sublayer(part, y, *args):
        if part.can_overwrite:
            part.forward(*args, accumulate=False)
        else:                                  # a part that can only add: into zeros
            y.zero_()
            part.forward(*args)


class ScaledPreNormBlock(Arrangement):
    joins_pending = True             # takes over a join that the layer before left for the next norm

    def __init__(self, spec):
        super().__init__(spec)
        self.mult = float(self.param("residual_mult", 1.0))

    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        y = ctx.buffer("sublayer.out", tuple(x.shape), torch.float32)
        h = self._norm(layer.norm1, x, ctx)
        ctx.note("ln1", h)
        SandwichNormBlock._sublayer(layer.mixer, y, h, y, ctx, cache, owns_cache)
        ctx.pending_join = (x, y, self.mult)
        if ctx.trace is not None:
            ctx.flush_join()
            ctx.note("res1", x)
        if not isinstance(layer.feed_forward, NoFeedForward):
            h = self._norm(layer.norm2, x, ctx)
            ctx.note("ln2", h)
            SandwichNormBlock._sublayer(layer.feed_forward, y, h, y, ctx)
            ctx.pending_join = (x, y, self.mult)
        if ctx.trace is not None:
            ctx.flush_join()
            ctx.note("res2", x)

    @staticmethod
    def _norm(norm, x, ctx):
        """The normed stream, with what is still to be added to the stream added by the same launch."""
        if isinstance(norm, RmsNorm) and norm.offset == 0.0 and norm.scale == 1.0 and x.stride(1) == 1:
            pending, ctx.pending_join = ctx.pending_join, None
            if pending is not None and pending[0] is not x:
                ctx.pending_join = pending
                ctx.flush_join()
                pending = None
            out = ctx.buffer("stream.normed", tuple(x.shape), norm.runtime.dtype)
            y, mult = (pending[1], pending[2]) if pending is not None else (None, 0.0)
            return norm.runtime.ops.residual_add_norm(x, y, mult, norm.weight, norm.eps, out)
        ctx.flush_join()
        return norm.forward(x)


class ParallelPreNormBlock(Arrangement):
    def forward(self, x, layer, ctx, cache, owns_cache: bool) -> None:
        n1, n2 = layer.norm1, layer.norm2
        alone = isinstance(layer.feed_forward, NoFeedForward)
        if (not alone and type(n1) is RmsNorm and type(n2) is RmsNorm and n1.eps == n2.eps and x.stride(1) == 1
                and n1.offset == n2.offset == 0.0 and n1.scale == n2.scale == 1.0):
            dt = n1.runtime.dtype
            h1 = ctx.buffer("stream.normed", tuple(x.shape), dt)
            h2 = ctx.buffer("stream.normed2", tuple(x.shape), dt)
            n1.runtime.ops.rms_norm_pair(x, n1.weight, n2.weight, n1.eps, h1, h2)
        else:
            h1 = n1.forward(x)
            h2 = None if alone else n2.forward(x)         # before the mixer changes x
        ctx.note("ln1", h1)
        layer.mixer.forward(h1, x, ctx, cache, owns_cache)
        ctx.note("res1", x)
        if not alone:
            ctx.note("ln2", h2)
            layer.feed_forward.forward(h2, x, ctx)
        ctx.note("res2", x)


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
register_part("arrangement", "parallel_pre_norm", ParallelPreNormBlock, replace=True)
register_part("arrangement", "scaled_pre_norm", ScaledPreNormBlock, replace=True)
register_part("arrangement", "sandwich_norm", SandwichNormBlock, replace=True)
