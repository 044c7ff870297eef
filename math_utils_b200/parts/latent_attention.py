"""Attention through a shared low-rank latent.

Parameters: ``hidden_size, n_heads, dim`` (unrotated query/key entries per head), ``rot_dim`` (rotated
entries per head), ``vdim`` (value entries per head), ``kv_rank`` (latent size), ``softmax_scale``,
``eps`` (of the latent's RMS norm), ``rot`` = {base, dims, scaling?} and ``own_kv`` (false for a layer
that reads the latent cache of an earlier layer and has no down-projection of its own).

Per token the layer keeps ONE row for all heads: the RMS-normed latent c (kv_rank values) and one
rotated key part (rot_dim values).  With k_h = U_h c and v_h = V_h c the score of head h is
    (q_h^n . U_h c + q_h^r . k^r) * scale = ((U_h^T q_h^n) . c + q_h^r . k^r) * scale
and the head's output V_h (sum_j p_j c_j), so the attention itself runs in latent space over the
cached rows, the same rows for every head, and the two up-projections become products per head before
and after it: keys and values are never expanded.  An output gate sigmoid(G h) multiplies the
concatenated heads before the output projection.

Switches for other designs, each with its constants: ``q_rank`` r_q > 0 sends the queries through a latent of
their own, q = U_q rmsnorm(D_q h) (tensors ``dq`` [r_q, hidden], ``dq_norm`` [r_q], ``uq`` [heads * (dim + rot_dim),
r_q] instead of ``q``; the norm's eps is ``eps``); ``gate`` false leaves the output gate out (no ``gate`` tensor);
``sink`` adds exp(s_h) to head h's softmax denominator, s a learned number per head (tensor ``sink`` [heads]) that
is not scaled and has no value behind it; ``rot_layout`` ``"pairs"`` turns entry 2i with entry 2i + 1 instead of
entry i with entry i + dims/2; ``exact_weights`` keeps the softmax's weights at some 16 bits where the tensor-core
kernel multiplies them with the latents (two bfloat16 terms a weight), for designs that want them at 32 bits.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, RowCacheSpec, TensorSpec, register_part
from .linear import Linear
from .position import rotary_frequencies


class LatentAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads = int(p("hidden_size")), int(p("n_heads"))
        self.dim, self.rot_dim, self.vdim, self.kv_rank = int(p("dim")), int(p("rot_dim")), int(p("vdim")), int(p("kv_rank"))
        self.scale, self.eps = float(p("softmax_scale")), float(p("eps"))
        self.own_kv = bool(p("own_kv", True))
        self.window = int(p("window", 0))
        self.q_rank = int(p("q_rank", 0))
        self.has_gate, self.has_sink = bool(p("gate", True)), bool(p("sink", False))
        self.exact_weights = bool(p("exact_weights", False))
        self.rot_layout = p("rot_layout", "half")
        if self.rot_layout not in ("half", "pairs"):
            raise ConfigError(f"latent_attention: rot_layout '{self.rot_layout}' is not 'half' or 'pairs'")
        rot = p("rot")
        self.rot_dims = int(rot["dims"])
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ConfigError(f"latent_attention: {self.rot_dims} rotated entries do not fit the rotated part of {self.rot_dim}")
        self.freqs, self.magnitude = rotary_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
        self.q_head = self.dim + self.rot_dim
        self.row = self.kv_rank + self.rot_dim

    def tensor_specs(self):
        H, D, r = self.n_heads, self.hidden_size, self.kv_rank
        name = self.tensor_name
        if self.q_rank:
            specs = [TensorSpec(name("dq"), (self.q_rank, D)),
                     TensorSpec(name("dq_norm"), (self.q_rank,), role="vector", init="norm_weight"),
                     TensorSpec(name("uq"), (H * self.q_head, self.q_rank))]
        else:
            specs = [TensorSpec(name("q"), (H * self.q_head, D))]
        if self.own_kv:
            specs += [TensorSpec(name("dkv"), (self.row, D)),
                      TensorSpec(name("dkv_norm"), (r,), role="vector", init="norm_weight")]
        specs += [TensorSpec(name("uk"), (H * self.dim, r)), TensorSpec(name("uv"), (H * self.vdim, r))]
        if self.has_gate:
            specs.append(TensorSpec(name("gate"), (H * self.vdim, D)))
        if self.has_sink:
            specs.append(TensorSpec(name("sink"), (H,), role="vector", init="bias"))
        specs.append(TensorSpec(name("out"), (D, H * self.vdim), init="residual_projection"))
        return specs

    def cache_spec(self):
        return RowCacheSpec(self.row, self.window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        H = self.n_heads
        # one product for everything that reads the layer's input: queries (or their latent) | gate | down-projection,
        # each block padded with rows of zeros to a whole number of 16-byte pieces
        parts, self.at = [], {}
        for role, present in (("dq" if self.q_rank else "q", True), ("gate", self.has_gate), ("dkv", self.own_kv)):
            if not present:
                continue
            w = t(role)
            self.at[role] = len(parts) + 1
            parts.append(w)
            pad = -w.shape[0] % 8
            if pad:
                parts.append(torch.zeros((pad, self.hidden_size), dtype=w.dtype, device=w.device))
        self.widths = tuple(w.shape[0] for w in parts)
        self.proj = Linear(torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0], None, runtime)
        if self.q_rank:
            self.q_norm_weight = t("dq_norm")
            self.q_up_proj = Linear(t("uq"), None, runtime)
        self.sink = t("sink").contiguous() if self.has_sink else None
        self.norm_weight = t("dkv_norm") if self.own_kv else None
        # U_h^T as [kv_rank, dim] per head ([out, in] for the product that carries a query into latent space)
        self.q_up = t("uk").reshape(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()      # [H, kv_rank, dim]
        self.v_up = t("uv").reshape(H, self.vdim, self.kv_rank).contiguous()                     # [H, vdim, kv_rank]
        self.out = Linear(t("out"), None, runtime)
        # (one entry at least, so that the kernels always get a table)
        self.freq_table = torch.tensor(self.freqs or [0.0], dtype=torch.float64).to(torch.float32).to(runtime.device)

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T, H, r = ctx.n_tokens, self.n_heads, self.kv_rank
        views = ctx.buffer("latent.proj", (T, sum(self.widths)), dt, columns=self.widths)
        proj = views[0]
        gate = views[self.at["gate"]] if self.has_gate else None
        self.proj(h, out=proj)
        ctx.note("proj", proj)
        if self.q_rank:
            # the queries' latent, normed in float32, then up to the heads
            cq = ctx.buffer("latent.cq", (T, self.q_rank), dt)
            ops.rms_norm(views[self.at["dq"]], self.q_norm_weight, self.eps, out=cq)
            q = ctx.buffer("latent.q_heads", (T, H * self.q_head), dt)
            self.q_up_proj(cq, out=q)
        else:
            q = views[self.at["q"]]
        table = ctx.block_tables[cache.group]
        if owns_cache and not self.own_kv:
            raise ConfigError("a latent-attention layer without a down-projection cannot own a cache")
        # queries in latent space, float32: [T, H, kv_rank | rot_dim]
        qa = ctx.buffer("latent.q", (T, H * self.row), torch.float32)
        # one launch: this step's cache rows (norm, rotation) and the rotated part of the queries
        rotated = (q[:, self.dim:], self.q_head, qa[:, r:], self.row, H) if self.rot_dim else None
        if owns_cache or rotated is not None:
            ops.latent_append(views[self.at["dkv"]] if owns_cache else None, self.norm_weight, self.eps, self.freq_table,
                              self.magnitude, self.rot_dims, r, self.rot_dim, ctx.tok_pos, ctx.tok_seq, table,
                              cache.page_tokens, cache.pages, queries=rotated, pairs=self.rot_layout == "pairs")
        ops.heads_gemm(q, self.q_up, qa, self.q_head, self.row)
        ctx.note("q_latent", qa)
        mixed = ctx.buffer("latent.mixed", (T, H * r), dt)
        n_splits, part_o, part_ml = self.splits(ctx)
        ops.latent_attention(qa, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq, H, r, self.scale,
                             mixed, n_splits, part_o, part_ml, tiles=ctx.q_tiles, single_tokens=ctx.is_decode,
                             sink=self.sink, two_term_weights=self.exact_weights)
        ctx.note("mixed", mixed)
        heads = ctx.buffer("latent.heads", (T, H * self.vdim), dt)
        ops.heads_gemm(mixed, self.v_up, heads, r, self.vdim, gate=gate)
        ctx.note("attn", heads)
        self.out(heads, residual=residual if accumulate else None, out=residual)

    def splits(self, ctx):
        """Single-token steps cut each sequence's rows into parts so that the blocks fill the GPU; a part is never
        shorter than 128 rows of the longest sequence the step may hold."""
        if not ctx.is_decode:
            return 1, None, None
        items = ctx.n_tokens * self.n_heads
        tc = self.runtime.dtype == torch.bfloat16 and self.runtime.ops.LATENT_TC
        blocks = ctx.n_tokens * -(-self.n_heads // 32) if tc else items      # the tensor-core kernel: 32 heads a block
        by_fill = -(-((2 if tc else 4) * self.runtime.ops.sm_count(self.runtime.device)) // blocks)
        n = max(1, min(by_fill, -(-ctx.max_kv_len // 128), 32))
        if n == 1:
            return 1, None, None
        return n, ctx.scratch("latent_part_o", items * n * self.kv_rank), ctx.scratch("latent_part_ml", items * n * 2)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
