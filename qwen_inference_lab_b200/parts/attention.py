"""Causal grouped-query attention over paged keys and values.

Per token: q, k, v projections (one stacked product), RMSNorm of every q and k
head over head_dim, rotation of q and k by the token's absolute position, k and v
written to the request's pages, softmax(q k^T * scale) over the keys up to the
token's own position (inside the window, if one is set), times v, then the output
projection (qil/model.py:48-69 for a chunk, :73-84 for single tokens; both are
the same computation here, every token of the flat batch takes it).  Query head
``h`` reads kv head ``h // (n_q_heads // n_kv_heads)`` (qil/paged_attention.py:21).

Options for designs without rotation: a bias that grows with distance taken off the scaled score
(``distance_slopes``, one slope per query head: score = q.k * scale - slope_h * (i - j)), a query
temperature that grows with the logarithm of the position (``q_temperature`` = (coef, every):
q_p * (1 + coef * ln(floor((p + 1) / every) + 1))), and value heads of another size than key heads
(``v_head_dim``).  Further options, each with its constants as arguments:

``conv_taps``      a short causal convolution over time on every channel of q, k and v right after the
                   projection (weights ``<q|k|v><conv suffix>`` [channels, taps]); the last taps - 1 projected rows
                   of a request are kept in a state slot beside its pages
``softcap``        score <- cap * tanh(score / cap) on the scaled product, before any bias
``distance_bias``  (rows, farthest): a learned table [rows, query heads] (``names["distance_bias"]``) added to the
                   score by distance: one row per distance below rows / 2, then rows that grow with the logarithm
                   of the distance up to ``farthest``, the last row for everything beyond (``distance_rows``)
``chunk``          position i sees the keys j <= i of its own chunk only: floor(i / chunk) = floor(j / chunk)
``sink``           one is added to the softmax's denominator (a key of score zero without a value); ``"learned"``:
                   exp(s_h) is added instead, s_h a learned score per query head (``names["sink"]``) that is not scaled

A rotation whose angles the kernels compute from frequencies (``position`` a :class:`RotaryFrequencies`: either
layout, on the first dimensions of a head only if so wished) and ``whole_qk_norm_eps`` (q and k are each divided by
their root mean square over the whole projection, all heads at once, and multiplied by a weight per element
``names["q_norm"]``, ``names["k_norm"]``, before the rotation) go with every option above but the per-head norms,
the short convolution and the query temperature.  With such a rotation ``qk_norm_eps`` norms every head by itself
(one weight of head_dim for all query heads, one for all key heads) in the same kernel.  ``values_from_keys``: there
is no value projection; a position's value is its key as projected, before norm and rotation.  ``head_gate``: the
name of a [query heads, hidden] matrix G; head h's output is multiplied by sigmoid(G x)_h before the output
projection (G's rows ride behind the keys' in the stacked projection).
"""
from __future__ import annotations

import math

import torch

from ..kernels import attention_mma, gemm_tc, ops
from .base import KVCacheSpec, Mixer, Param, StateSpec, StepPlanner
from .linear import Linear, StackedLinear
from .rotary import RotaryFrequencies


class PagedAttentionPlanner(StepPlanner):
    """The host hook of the attention mixers: a step's segments cut into the query tiles and the list
    of single tokens that the attention kernels take (``attention_mma.describe_segments``).  All
    attention layers of a model share the one plan."""
    key = attention_mma.PLAN_KEY

    def plan(self, segments):
        return attention_mma.describe_segments(segments.first, segments.starts, segments.lens, segments.rows)

    def refresh_single_tokens(self, arrays, segments):
        attention_mma.refresh_single_tokens(arrays, segments.starts)
        return True


_PLANNER = PagedAttentionPlanner()


def distance_rows(rows: int, farthest: int, count: int) -> list:
    """The row of a distance table with ``rows`` rows for each distance 0 .. count - 1: the distance itself below
    half = rows // 2, else min(rows - 1, half + floor(ln(n / half) / ln(farthest / half) * (rows - half)))."""
    half = rows // 2
    if rows < 2 or farthest <= half:
        raise ValueError(f"a distance table of {rows} rows needs a farthest distance beyond {half}, not {farthest}")
    result = []
    for n in range(count):
        if n < half:
            result.append(n)
        else:
            result.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(farthest / half) * (rows - half)))))
    return result


class GroupedQueryAttention(Mixer):
    """Sizes and constants are arguments; ``names`` gives the checkpoint names.

    names: dict with keys q, k, v, o (projection names, without ``.weight``) and,
    when ``qk_norm_eps`` is not None, q_norm and k_norm.
    ``reads_shared_cache=True`` builds a layer without k and v projections that
    attends over pages another layer wrote (the model's order says which).
    """
    graph_safe = True

    def __init__(self, hidden_size, n_q_heads, n_kv_heads, head_dim, *, names, bias=False,
                 qk_norm_eps=None, position=None, window=0, scale=None, reads_shared_cache=False,
                 v_head_dim=None, distance_slopes=None, q_temperature=None, out_bias=None,
                 suffixes=(".weight", ".bias"), conv_taps=0, conv_suffix=".conv", softcap=0.0, distance_bias=None,
                 chunk=0, sink=False, whole_qk_norm_eps=None, norm_suffix=".weight", values_from_keys=False,
                 head_gate=None):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads do not divide into {n_kv_heads} kv heads")
        self.hidden_size, self.head_dim = int(hidden_size), int(head_dim)
        self.n_q_heads, self.n_kv_heads = int(n_q_heads), int(n_kv_heads)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.qk_norm_eps = qk_norm_eps
        self.position = position
        self.reads_shared_cache = bool(reads_shared_cache)
        self.v_head_dim = int(v_head_dim) if v_head_dim else self.head_dim
        self.distance_slopes = None if distance_slopes is None else [float(v) for v in distance_slopes]
        if self.distance_slopes is not None and len(self.distance_slopes) != self.n_q_heads:
            raise ValueError("distance_slopes needs one slope per query head")
        self.q_temperature = None if not q_temperature else (float(q_temperature[0]), int(q_temperature[1]))
        if self.q_temperature is not None and self.q_temperature[1] < 1:
            raise ValueError("the query temperature's step must be a positive number of positions")
        self.conv_taps, self.softcap, self.chunk, self.sink = int(conv_taps), float(softcap or 0.0), int(chunk or 0), bool(sink)
        self.learned_sink = sink == "learned"
        self.whole_qk_norm_eps = None if whole_qk_norm_eps is None else float(whole_qk_norm_eps)
        # the projection's tail is the kernel that norms over the whole projection and rotates by frequencies
        self.frequency_tail = isinstance(position, RotaryFrequencies) or self.whole_qk_norm_eps is not None
        if self.frequency_tail and (conv_taps or q_temperature is not None
                                    or (qk_norm_eps is not None and self.whole_qk_norm_eps is not None)
                                    or (position is not None and not isinstance(position, RotaryFrequencies))):
            raise ValueError("rotation from frequencies and the norm over the whole projection go without a rotary "
                             "table, a short convolution or a query temperature, and with one kind of q/k norm")
        self.values_from_keys, self.head_gate = bool(values_from_keys), head_gate
        if (self.values_from_keys or head_gate) and not self.frequency_tail:
            raise ValueError("keys as values and a gate per head go with the rotation from frequencies")
        if self.values_from_keys and (reads_shared_cache or (v_head_dim and int(v_head_dim) != int(head_dim))):
            raise ValueError("keys as values need keys of the layer's own, and values as large as keys")
        if isinstance(position, RotaryFrequencies) and position.rotary_dim > self.head_dim:
            raise ValueError(f"{position.rotary_dim} rotated dimensions in heads of {self.head_dim}")
        if self.conv_taps < 0 or self.softcap < 0 or self.chunk < 0:
            raise ValueError("taps, softcap and chunk size cannot be negative")
        self.distance_bias = None if not distance_bias else (int(distance_bias[0]), int(distance_bias[1]))
        self.modified_scores = bool(self.softcap or self.distance_bias or self.chunk or self.sink)
        if self.modified_scores and self.window:
            raise ValueError("a window does not go with chunks, a softcap, a distance table or a sink")
        # without per-head norms and rotation the projection's tail is a copy (times the temperature) and the page write
        self.plain_tail = (self.v_head_dim != self.head_dim or self.distance_slopes is not None
                           or self.q_temperature is not None or self.conv_taps > 0 or self.modified_scores)
        if self.conv_taps and self.q_temperature is not None:
            raise ValueError("the short convolution goes without a query temperature")
        if self.plain_tail and not self.frequency_tail and (qk_norm_eps is not None or position is not None):
            raise ValueError("distance slopes, query temperature and a value size of its own go without q/k norms and rotation")
        self._slopes = self._slopes_log2 = None
        pieces = [(names["q"], n_q_heads * head_dim)]
        if not self.reads_shared_cache:
            pieces += [(names["k"], n_kv_heads * head_dim)]
            if not self.values_from_keys:
                pieces += [(names["v"], n_kv_heads * self.v_head_dim)]
        if head_gate:
            pieces += [(head_gate, n_q_heads)]
        self.qkv = StackedLinear(hidden_size, pieces, bias=bias, suffixes=suffixes)
        self.out = Linear(n_q_heads * self.v_head_dim, hidden_size, name=names["o"],
                          bias=bias if out_bias is None else out_bias, suffixes=suffixes)
        self._extra = {}
        self.conv = None
        if self.conv_taps:
            self.conv = [Param((rows, self.conv_taps), std=0.5) for _, rows in pieces]
            for (name, _), param in zip(pieces, self.conv):
                self._extra[name + suffixes[0] + conv_suffix] = param
        self.distance_table = None
        if self.distance_bias is not None:
            distance_rows(self.distance_bias[0], self.distance_bias[1], 1)      # refuses constants that do not fit
            self.distance_table = Param((self.distance_bias[0], self.n_q_heads), std=0.5)
            self._extra[names["distance_bias"]] = self.distance_table
        self.sink_logits = None
        if self.learned_sink:
            self.sink_logits = Param((self.n_q_heads,), std=1.0)
            self._extra[names["sink"]] = self.sink_logits
        self.whole_q_norm = self.whole_k_norm = None
        if self.whole_qk_norm_eps is not None:
            self.whole_q_norm = Param((n_q_heads * head_dim,), init="norm", std=0.05)
            self._extra[names["q_norm"] + norm_suffix] = self.whole_q_norm
            if not self.reads_shared_cache:
                self.whole_k_norm = Param((n_kv_heads * head_dim,), init="norm", std=0.05)
                self._extra[names["k_norm"] + norm_suffix] = self.whole_k_norm
        self._conv_w = self._bias_by_distance = self._options = self._sinks = None
        self.q_norm = self.k_norm = None
        self._norm_names = None
        if qk_norm_eps is not None:
            self.q_norm = Param((head_dim,), init="norm", std=0.05)
            self.k_norm = Param((head_dim,), init="norm", std=0.05)
            self._norm_names = (names["q_norm"] + norm_suffix, names["k_norm"] + norm_suffix)

    def named_params(self):
        if self._norm_names is None:
            return dict(self._extra)
        return {self._norm_names[0]: self.q_norm, self._norm_names[1]: self.k_norm, **self._extra}

    def children(self):
        parts = [self.qkv, self.out]
        if self.position is not None:
            parts.append(self.position)
        return parts

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        if self.q_norm is not None and self.q_norm.data.dtype != self.k_norm.data.dtype:
            self.q_norm.data, self.k_norm.data = self.q_norm.data.float(), self.k_norm.data.float()
        if self.distance_slopes is not None:
            self._slopes = torch.tensor(self.distance_slopes, dtype=torch.float32, device=device)
            self._slopes_log2 = (self._slopes.double() * 1.4426950408889634).float().contiguous()
        if self.conv is not None:
            self._conv_w = torch.cat([p.data for p in self.conv], dim=0).t().contiguous()     # [taps, channels]
            for p in self.conv:
                p.data = None
        if self.distance_table is not None:
            # the table by distance, one row per query head: the kernels look a distance up, not a bucket; every
            # distance from the first one of the last row on reads the last entry, and a chunk bounds the distances
            rows, farthest = self.distance_bias
            of_distance = distance_rows(rows, farthest, farthest + 1)
            count = of_distance.index(rows - 1) + 1
            if self.chunk:
                count = max(1, min(count, self.chunk))
            index = torch.tensor(of_distance[:count], dtype=torch.long, device=self.distance_table.data.device)
            self._bias_by_distance = self.distance_table.data.float()[index].t().contiguous()
        if self.sink_logits is not None:           # the softmax runs in float32 whatever the activations are
            self._sinks = self.sink_logits.data.float().contiguous()
        if self.whole_q_norm is not None and self.whole_k_norm is not None \
                and self.whole_q_norm.data.dtype != self.whole_k_norm.data.dtype:
            self.whole_q_norm.data, self.whole_k_norm.data = self.whole_q_norm.data.float(), self.whole_k_norm.data.float()
        self._options = attention_mma.ScoreOptions(self.softcap, self._bias_by_distance, self.chunk, self.sink,
                                                   sink_logits=self._sinks)

    def step_planners(self):
        return {**super().step_planners(), _PLANNER.key: _PLANNER}

    def cache_spec(self):
        """Pages for keys and values; with a short convolution also a state slot for the projected rows that the
        next step's first tokens reach back to (a pair of specs: the view is then a pair too)."""
        pages = None if self.reads_shared_cache else KVCacheSpec(
            self.n_kv_heads, self.head_dim, self.window, self.v_head_dim if self.v_head_dim != self.head_dim else 0,
            chunk=self.chunk)
        if self.conv_taps > 1:
            if self.reads_shared_cache:
                raise ValueError("a layer with a short convolution keeps keys and values of its own")
            return (pages, StateSpec((self.conv_taps - 1, self.qkv.out_features), torch.float32))
        return pages

    takes_norm = True

    @property
    def takes_out_scale(self):
        return self.plain_tail or self.frequency_tail

    def forward(self, ctx, x, cache, residual=None, norm=None, out_scale=None, out_float32=False):
        """x [N, hidden] -> [N, hidden] (+ residual).  ``cache`` is a KVCacheView (with a short convolution: a
        pair of it and a StateView).  With ``norm`` x is the block's un-normed input and the first projection
        applies the norm."""
        n = x.shape[0]
        n_kv = 0 if self.reads_shared_cache else self.n_kv_heads
        if self.frequency_tail:
            qkv = self.qkv.forward(ctx, x, norm=norm)
            q = ctx.empty((n, self.n_q_heads * self.head_dim))
            q_width, k_width = self.n_q_heads * self.head_dim, n_kv * self.head_dim
            rotation = self.position
            per_head = self.q_norm is not None
            q_weight = self.q_norm if per_head else self.whole_q_norm
            k_weight = self.k_norm if per_head else self.whole_k_norm
            # keys as values: the value rows are copied from the keys' columns, as projected
            v_column = q_width if self.values_from_keys else q_width + k_width
            ops.qk_rotate_store(qkv, (0, q_width, v_column), q, cache.pages,
                                q_weight.data if q_weight is not None else None,
                                k_weight.data if k_weight is not None else None,
                                (self.qk_norm_eps if per_head else self.whole_qk_norm_eps) or 0.0,
                                rotation.freq if rotation is not None else None,
                                rotation.rotary_dim if rotation is not None else 0,
                                rotation.layout if rotation is not None else 0, ctx.positions, ctx.token_row,
                                cache.block_table, self.n_q_heads, n_kv, self.head_dim, self.v_head_dim, cache.page_size,
                                per_head=per_head)
            attended = ctx.empty((n, self.n_q_heads * self.v_head_dim))
            self._attend(ctx, q, cache, attended)
            if self.head_gate:
                ops.head_gate(attended, self.v_head_dim, qkv, qkv.shape[1] - self.n_q_heads)
            return self.out.forward(ctx, attended, residual=residual, out_scale=out_scale, out_float32=out_float32)
        if out_float32:
            raise ValueError("a float32 result is given by the layers that rotate by frequencies only")
        if self.plain_tail:
            qkv = self.qkv.forward(ctx, x, norm=norm)
            q = ctx.empty((n, self.n_q_heads * self.head_dim))
            if self.conv_taps:
                state = None
                if self.conv_taps > 1:
                    cache, state = cache
                    state = state.slots
                else:
                    state = torch.empty((1, 0, qkv.shape[1]), dtype=torch.float32, device=qkv.device)
                ops.short_conv_store(qkv, self._conv_w, state, q, cache.pages, ctx.positions, ctx.token_row,
                                     cache.block_table, ctx.seg_row, ctx.seg_start, ctx.seg_len, ctx.n_segments,
                                     self.n_q_heads, n_kv, self.head_dim, self.v_head_dim, cache.page_size)
            else:
                coef, every = self.q_temperature or (0.0, 0)
                ops.qkv_store(qkv, q, cache.pages, ctx.positions, ctx.token_row, cache.block_table, self.n_q_heads,
                              n_kv, self.head_dim, self.v_head_dim, cache.page_size, coef, every)
            attended = ctx.empty((n, self.n_q_heads * self.v_head_dim))
            self._attend(ctx, q, cache, attended)
            return self.out.forward(ctx, attended, residual=residual, out_scale=out_scale)
        if out_scale is not None:
            raise ValueError("an output scale is taken by the layers without q/k norms and rotation only")
        table = self.position.table if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        q_norm = self.q_norm.data if self.q_norm is not None else None
        k_norm = self.k_norm.data if self.k_norm is not None else None
        if gemm_tc.qkv_tail_usable(x, self.qkv._weight(), self.head_dim, rotary_dim, (q_norm, k_norm), cache.pages):
            # long prompt portions: one tcgen05 kernel projects, norms, rotates and writes the pages
            if norm is not None:
                x = norm.forward(ctx, x)
            q = ctx.empty((n, self.n_q_heads * self.head_dim))
            gemm_tc.gemm_tc_qkv(x, self.qkv._weight(), self.qkv._bias(), q, cache.pages, table, q_norm, k_norm,
                                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, ctx.positions,
                                ctx.token_row, cache.block_table, self.n_q_heads, n_kv, cache.page_size)
            attended = ctx.empty((n, self.n_q_heads * self.head_dim))
            self._attend(ctx, q, cache, attended)
            return self.out.forward(ctx, attended, residual=residual)
        qkv = self.qkv.forward(ctx, x, norm=norm)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if attention_mma.projection_tail_usable(ctx, qkv, cache, self.n_q_heads, self.n_kv_heads, self.head_dim,
                                                rotary_dim, (q_norm, k_norm)):
            # a step of single tokens: the attention kernel norms, rotates and stores what it needs itself
            attended = ctx.empty((n, self.n_q_heads * self.head_dim))
            attention_mma.attend_projection(ctx, qkv, cache, attended, self.n_q_heads, self.n_kv_heads, n_kv,
                                            self.head_dim, self.window, self.scale, q_norm, k_norm, eps, table,
                                            rotary_dim)
            return self.out.forward(ctx, attended, residual=residual)
        q = ctx.empty((n, self.n_q_heads * self.head_dim))
        ops.qk_norm_rope_store(qkv, q, cache.pages, q_norm, k_norm, eps, table, rotary_dim, ctx.positions,
                               ctx.token_row, cache.block_table, self.n_q_heads, n_kv, self.head_dim, cache.page_size)
        attended = ctx.empty((n, self.n_q_heads * self.head_dim))
        self._attend(ctx, q, cache, attended)
        return self.out.forward(ctx, attended, residual=residual)

    def _attend(self, ctx, q, cache, out):
        tensor_cores = q.dtype == torch.bfloat16 and self.v_head_dim == self.head_dim \
            and attention_mma.supports(self.head_dim, self.n_q_heads, self.n_kv_heads)
        if self.modified_scores and tensor_cores:
            attention_mma.attend(ctx, q, cache, out, self.n_q_heads, self.n_kv_heads, self.head_dim, 0, self.scale,
                                 self._slopes_log2, self._options)
            return
        if self.modified_scores:
            ops.attention_generic(q, cache.pages, out, ctx.positions, ctx.token_row, cache.block_table,
                                  self.n_q_heads, self.n_kv_heads, self.head_dim, cache.page_size,
                                  self.window, self.scale, v_dim=self.v_head_dim, slopes=self._slopes,
                                  softcap=self.softcap, distance_bias=self._bias_by_distance, chunk=self.chunk,
                                  sink=self.sink, sink_logits=self._sinks)
            return
        if q.dtype == torch.bfloat16 and self.v_head_dim == self.head_dim \
                and attention_mma.supports(self.head_dim, self.n_q_heads, self.n_kv_heads):
            attention_mma.attend(ctx, q, cache, out, self.n_q_heads, self.n_kv_heads, self.head_dim,
                                 self.window, self.scale, self._slopes_log2)
            return
        ops.attention_generic(q, cache.pages, out, ctx.positions, ctx.token_row, cache.block_table,
                              self.n_q_heads, self.n_kv_heads, self.head_dim, cache.page_size,
                              self.window, self.scale, v_dim=self.v_head_dim, slopes=self._slopes)
