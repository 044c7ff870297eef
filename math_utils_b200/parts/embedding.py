"""Token embedding: a row of the table per token (times the parameter
``scale``, 1 if absent), plus the position table's row when the position
encoding has one; the result is the float32 residual stream
(include/ai/LocalModel.hpp:3686-3697).  Heads: ``tied_head`` (the token table
itself) and ``linear_head`` (a matrix of its own, no bias)."""
from __future__ import annotations

from ..config.base import PartSpec
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))
        self.scale = float(self.param("scale", 1.0))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.vocab_size, self.hidden_size), role="table"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def table(self):
        return self.weight

    def forward(self, ctx, position_table):
        return self.runtime.ops.embed(ctx.token_ids, ctx.tok_pos, self.weight, position_table, scale=self.scale)


class TokenPairEmbedding(Embedding):
    """A row per token plus a row of a second table chosen by the token and the one before it:
    row (previous * mul_prev + token * mul_cur) mod buckets, and row ``buckets`` (the table's last) for the first
    token of a sequence.  The token before the first token of a step is the sequence's state: the cache keeps
    it per slot (``StepContext.last_tokens``), and the kernel moves it on."""
    keeps_last_token = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))
        self.buckets = int(self.param("buckets"))
        self.mul_prev, self.mul_cur = int(self.param("mul_prev")), int(self.param("mul_cur"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.vocab_size, self.hidden_size), role="table"),
                TensorSpec(self.tensor_name("pair_weight"), (self.buckets + 1, self.hidden_size), role="table"))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]
        self.pair_weight = tensors[self.tensor_name("pair_weight")]

    def table(self):
        return self.weight

    def forward(self, ctx, position_table):
        if position_table is not None:
            raise ValueError("the token-pair embedding adds no position table")
        if ctx.last_tokens is None or ctx.seq_first is None:
            raise ValueError("the token-pair embedding needs the cache's last tokens and the step's sequence starts")
        import torch
        # in bfloat16 the same launch leaves the rows rounded too, for a first sublayer that reads the stream itself
        copy = (ctx.buffer("stream.copy", (ctx.n_tokens, self.hidden_size), torch.bfloat16)
                if self.runtime.dtype == torch.bfloat16 else None)
        x = self.runtime.ops.embed_pair(ctx.token_ids, ctx.tok_pos, ctx.tok_seq, ctx.seq_first, ctx.seq_slots,
                                        ctx.last_tokens, self.weight, self.pair_weight, self.mul_prev, self.mul_cur,
                                        ctx.is_decode, copy=copy)
        ctx.stream_copy = copy
        return x


class TiedHead(Head):
    """Logits = h @ table^T with the token table itself, no bias
    (include/ai/LocalModel.hpp:1938-1940, 3796-3799)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))
        self.linear = None

    def attach_embedding(self, embedding: Embedding) -> None:
        from .linear import Linear
        table = embedding.table()
        if tuple(table.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("the tied head and the token table disagree on their sizes")
        self.linear = Linear(table, None, self.runtime)

    takes_lazy_norm = True

    def forward(self, h):
        import torch
        return self.linear(h, out_dtype=torch.float32)


class LinearHead(Head):
    """Logits = h @ W^T with an output matrix ``weight`` [vocab, hidden] of its own, no bias.  With the
    parameter ``softcap`` c > 0 the logits become c * tanh(logits / c)."""
    takes_lazy_norm = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self.param("vocab_size"))
        self.hidden_size = int(self.param("hidden_size"))
        self.softcap = float(self.param("softcap", 0.0) or 0.0)

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.vocab_size, self.hidden_size), role="matrix"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        from .linear import Linear
        self.linear = Linear(tensors[self.tensor_name("weight")], None, runtime)

    def forward(self, h):
        import torch
        logits = self.linear(h, out_dtype=torch.float32)
        if self.softcap > 0.0:
            self.runtime.ops.softcap(logits, self.softcap)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("embedding", "token_pair_embedding", TokenPairEmbedding, replace=True)
register_part("head", "linear_head", LinearHead, replace=True)
register_part("head", "tied_head", TiedHead, replace=True)
