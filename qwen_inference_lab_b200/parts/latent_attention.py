"""Latent attention: keys and values of all heads grow out of one small latent per token, which is all the cache keeps.

Per token, with H heads, d plain and r rotated query/key dimensions per head, e value dimensions and a latent of c:

    q = Wq h                          [H][d plain, r rotated]
    (l, s) = Wdkv h                   c + r rows;  z = l / sqrt(mean(l^2) + eps) * w  (float32);  s is one rotated key
                                      part shared by all heads
    key of head a   = [Wuk_a z, rot(s)]      value of head a = Wuv_a z
    score           = (q_plain . Wuk_a z + rot(q_rot) . rot(s)) * scale,  softmax inside a sliding window
    y = Wo concat_a( sigmoid(Wg h)_a * sum_j p_j Wuv_a z_j )

Only z and rot(s) are cached: the products with Wuk and Wuv are moved to the query's side.  q_plain . (Wuk_a z) =
(Wuk_a^T q_plain) . z, so the query of head a becomes [Wuk_a^T q_plain, rot(q_rot)] of c + r numbers, every head reads
the same key row [z, rot(s)] (attention with one key/value head), the weighted sum runs over the z_j, and Wuv_a is
applied once to that sum.  Kernels: the stacked projection (q, dkv, g); ``ops.latent_prepare`` (norm of the latent,
the rotations, the page write); ``ops.head_product`` (the query through Wuk^T); the engine's paged attention with a
window; ``ops.head_product`` again (the sum through Wuv, times the gate); the output product.  A bfloat16 step of more
than ``LIBRARY_ROWS`` tokens hands the two per-head products to the library as batched products over strided views
of the same buffers (as ``Linear`` does with its products), and ``ops.head_gate`` applies the gates.

Options for other designs of the same mixer: no rotated part at all (``rot_dim`` 0, ``position`` None); queries that
come through a latent of their own (``query_latent``: c_q = rms(Wdq h) w, q = Wuq c_q, with Wdq's rows in the stacked
projection, the norm over that column range and Wuq a product of its own); a learned sink (``sink="learned"``: exp(s_a)
joins head a's denominator; no window then); a gate per output element instead of one per head (``gate="element"``).

A page holds one row per token, the key [z, rot(s)]; the token's value z is that row's first c columns (the cache's
shared rows), so the attention kernels fetch one tile per 64 positions and use it for the scores and for the
weighted sum alike.  Where c + r is a head size the tensor-core attention takes (a multiple of 16 up to 256) a
bfloat16 step runs there, and its output rows are c + r wide with the sums of the latents in their first c columns;
otherwise, and in float32, the float32 kernel runs and gives rows of c.
"""
from __future__ import annotations

import torch

from ..kernels import attention_mma, ops
from .attention import _PLANNER
from .base import KVCacheSpec, Mixer, Param
from .linear import Linear, StackedLinear
from .rotary import RotaryFrequencies


LIBRARY_ROWS = 64      # bfloat16 steps of more tokens than this run the per-head products as batched library products


class LatentAttention(Mixer):
    """names: dict with keys q, dkv, dkv_norm, uk, uv, g, o (tensor names; ``suffixes`` are appended to the
    projections', ``norm_suffix`` to the norms'); with ``query_latent`` (the latent's size) dq, dq_norm and uq in place of
    q; with a learned sink also sink.  ``position``: a :class:`RotaryFrequencies` over the rotated part."""
    graph_safe = True

    def __init__(self, hidden_size, n_heads, plain_dim, rot_dim, value_dim, latent_dim, *, scale, window, position,
                 norm_eps, names, suffixes=(".weight", ".bias"), norm_suffix=".weight", query_latent=0, sink=None,
                 gate="head"):
        self.hidden_size, self.n_heads = int(hidden_size), int(n_heads)
        self.plain_dim, self.rot_dim, self.value_dim, self.latent_dim = int(plain_dim), int(rot_dim), int(value_dim), int(latent_dim)
        self.scale, self.window, self.norm_eps = float(scale), int(window or 0), float(norm_eps)
        if self.rot_dim == 0 and position is None:
            pass                                       # keys without a rotated part: no positions at all
        elif not isinstance(position, RotaryFrequencies) or position.rotary_dim > self.rot_dim:
            raise ValueError("latent attention rotates by frequencies, over at most its rotated dimensions")
        if sink not in (None, "learned") or gate not in ("head", "element"):
            raise ValueError(f"latent attention: sink {sink!r} (None or 'learned'), gate {gate!r} ('head' or 'element')")
        if sink and self.window:
            raise ValueError("a sink goes without a window")
        self.query_latent, self.learned_sink, self.gate_each = int(query_latent or 0), sink == "learned", gate == "element"
        if self.query_latent and self.rot_dim:
            raise ValueError("queries through a latent go without a rotated part")
        self.position = position
        self.key_width = self.latent_dim + self.rot_dim
        # the width of a bfloat16 step's attended rows: see the module's text
        self.tensor_cores = attention_mma.supports(self.key_width, 1, 1)
        self.value_width = self.key_width if self.tensor_cores else self.latent_dim
        q_width = self.n_heads * (self.plain_dim + self.rot_dim)
        first = (names["dq"], self.query_latent) if self.query_latent else (names["q"], q_width)
        gates = self.n_heads * (self.value_dim if self.gate_each else 1)
        self.projection = StackedLinear(hidden_size, [first, (names["dkv"], self.key_width), (names["g"], gates)],
                                        suffixes=suffixes)
        self.columns = (0, first[1], first[1] + self.key_width)
        self.latent_norm = Param((self.latent_dim,), init="norm", std=0.05)
        self.key_up = Param((self.n_heads * self.plain_dim, self.latent_dim))
        self.value_up = Param((self.n_heads * self.value_dim, self.latent_dim))
        self._names = {names["dkv_norm"] + norm_suffix: self.latent_norm, names["uk"] + suffixes[0]: self.key_up,
                       names["uv"] + suffixes[0]: self.value_up}
        self.query_norm = self.query_up = self.sink_logits = None
        if self.query_latent:
            self.query_norm = Param((self.query_latent,), init="norm", std=0.05)
            self._names[names["dq_norm"] + norm_suffix] = self.query_norm
            self.query_up = Linear(self.query_latent, q_width, name=names["uq"], suffixes=suffixes)
        if self.learned_sink:
            self.sink_logits = Param((self.n_heads,), std=1.0)
            self._names[names["sink"]] = self.sink_logits
        self.out = Linear(self.n_heads * self.value_dim, hidden_size, name=names["o"], suffixes=suffixes)
        self._query_fold = self._value_unfold = self._options = self._sinks = None

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [part for part in (self.projection, self.query_up, self.out, self.position) if part is not None]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        common = self.projection._weight().dtype
        # per head: the query's plain part through Wuk_a^T [c, d]; the weighted sum of latents through Wuv_a [e, c]
        up = self.key_up.data.to(common).view(self.n_heads, self.plain_dim, self.latent_dim)
        self._query_fold = up.transpose(1, 2).contiguous()
        self._value_unfold = self.value_up.data.to(common).view(self.n_heads, self.value_dim, self.latent_dim).contiguous()
        self.key_up.data = self.value_up.data = None
        self.latent_norm.data = self.latent_norm.data.to(common).contiguous()
        if self.query_norm is not None:
            self.query_norm.data = self.query_norm.data.to(common).contiguous()
        if self.sink_logits is not None:           # the softmax runs in float32 whatever the activations are
            self._sinks = self.sink_logits.data.float().contiguous()
            self._options = attention_mma.ScoreOptions(sink_logits=self._sinks)

    def step_planners(self):
        return {**super().step_planners(), _PLANNER.key: _PLANNER}

    def cache_spec(self):
        return KVCacheSpec(1, self.key_width, self.window, self.latent_dim, shared_rows=True)

    def forward(self, ctx, x, cache, residual=None, out_float32=False):
        """x [N, hidden] -> [N, hidden] (+ residual); ``cache`` is a KVCacheView of rows [latent, rotated key part]."""
        projected = self.projection.forward(ctx, x)
        queries = self.prepare(ctx, projected, cache)
        attended = self.attend(ctx, queries, cache)
        mixed = self.expand(ctx, attended, projected)
        return self.out.forward(ctx, mixed, residual=residual, out_float32=out_float32)

    def _batched(self, projected):
        return projected.shape[0] > LIBRARY_ROWS and projected.dtype == torch.bfloat16 \
            and self._query_fold.dtype == torch.bfloat16

    def prepare(self, ctx, projected, cache):
        """The projection's tail: the token's key row into its page, the queries [N, H * (c + r)] as the attention
        reads them (plain part through Wuk^T, rotated part turned).  Queries that come through a latent of their own:
        the kernel that norms the key latent norms theirs too, their expansion is a product of its own."""
        n, heads, width = projected.shape[0], self.n_heads, self.key_width
        queries = ctx.empty((n, heads * width))
        rotation = self.position
        query_latent = ctx.empty((n, self.query_latent)) if self.query_latent else None
        ops.latent_prepare(projected, self.columns[0], self.columns[1], queries, cache.pages, self.latent_norm.data,
                           self.norm_eps, rotation.freq if rotation is not None else None,
                           rotation.rotary_dim if rotation is not None else 0,
                           rotation.layout if rotation is not None else 0, ctx.positions, ctx.token_row,
                           cache.block_table, heads, self.plain_dim, self.rot_dim, self.latent_dim, 0, cache.page_size,
                           query_latent=(self.columns[0], self.query_norm.data, query_latent) if self.query_latent else None)
        q_rows, q_width = projected, self.columns[1]
        if self.query_latent:
            q_rows = self.query_up.forward(ctx, query_latent)
            q_width = q_rows.shape[1]
        if self._batched(projected):
            plain = q_rows[:, :q_width].unflatten(1, (heads, self.plain_dim + self.rot_dim))[:, :, :self.plain_dim]
            torch.bmm(plain.transpose(0, 1), self._query_fold.transpose(1, 2),
                      out=queries.view(n, heads, width)[:, :, :self.latent_dim].transpose(0, 1))
        else:
            ops.head_product(q_rows, 0, self.plain_dim + self.rot_dim, self._query_fold, queries, 0, width)
        return queries

    def attend(self, ctx, queries, cache):
        """Every head over the one key row per token: per head a row whose first c columns are the weighted sum of
        latents, [N, H * (c + r)] from the tensor-core kernels and [N, H * c] from the float32 kernel."""
        n, heads, width = queries.shape[0], self.n_heads, self.key_width
        if queries.dtype == torch.bfloat16 and self.tensor_cores:
            attended = ctx.empty((n, heads * width))
            attention_mma.attend(ctx, queries, cache, attended, heads, 1, width, self.window, self.scale,
                                 options=self._options, shared_rows=True, value_cols=self.latent_dim)
        else:
            attended = ctx.empty((n, heads * self.latent_dim))
            ops.attention_generic(queries, cache.pages, attended, ctx.positions, ctx.token_row, cache.block_table, heads, 1,
                                  width, cache.page_size, self.window, self.scale, v_dim=self.latent_dim, shared_rows=True,
                                  sink=self.learned_sink, sink_logits=self._sinks)
        return attended

    def expand(self, ctx, attended, projected):
        """The weighted sums through Wuv, times the heads' gates: [N, H * e]."""
        n, heads = attended.shape[0], self.n_heads
        stride = attended.shape[1] // heads          # c + r or c: see ``attend``
        mixed = ctx.empty((n, heads * self.value_dim))
        if self._batched(projected):
            sums = attended.view(n, heads, stride)[:, :, :self.latent_dim]
            torch.bmm(sums.transpose(0, 1), self._value_unfold.transpose(1, 2),
                      out=mixed.view(n, heads, self.value_dim).transpose(0, 1))
            ops.head_gate(mixed, 1 if self.gate_each else self.value_dim, projected, self.columns[2])
        else:
            ops.head_product(attended, 0, stride, self._value_unfold, mixed, 0, self.value_dim,
                             gate=projected, gate_column=self.columns[2], gate_each=self.gate_each)
        return mixed
