"""Gated linear attention: a recurrent mixer whose state is a matrix per head, decayed per key channel.

Per head, with d key channels and e value channels, for the tokens of a sequence in order:

    a_t = sigmoid(A2 (A1 x_t) + b)^(1/tau)          decay per key channel, float32
    S_t = diag(a_t) S_(t-1) + k_t v_t^T              S_0 = 0, float32, one per request and layer call
    o_t = S_t^T (q_t * q_scale)
    y_t = W_o ( rmsnorm_e(o_t; w) * silu(W_g x_t) )  the norm is over a head's e values, w shared by heads

q, k, v, the gate and the low-rank input of the decay are one stacked product; the decays are a small kernel
of their own (``kernels.ops.gla_decay``); the recurrence, the norm and the gate are one kernel that walks a segment of the step from the request's state slot
(``kernels.ops.gla_scan``): single decoded tokens and prompt portions of up to ``LONG_SEGMENT`` tokens take it
token by token, and their result does not depend on the cut to the last bit.  Longer portions are cut into
chunks of ``CHUNK`` tokens that run side by side: every chunk's own state from zero, a carry over the chunks
in order, then every chunk again from its incoming state (twice the arithmetic, all chunks at once; the
carry rounds differently from the token-by-token scan, in the last bits).
"""
from __future__ import annotations

import torch

import numpy as np

from ..kernels import ops
from .base import Mixer, Param, StateSpec, StepPlanner
from .linear import Linear, StackedLinear

CHUNK = 64              # tokens of a chunk of a long segment
LONG_SEGMENT = 128      # segments longer than this are cut into chunks


class ScanPlanner(StepPlanner):
    """A step's segments as the scan wants them: the short ones as they are (first token, tokens, state slot),
    the long ones as chunks (first token, tokens, index among the step's chunks) and one carry entry per long
    segment (state slot, first chunk, chunks).  All recurrent layers of a model share the plan."""
    key = "state_scan"

    def plan(self, segments):
        lens = np.asarray(segments.lens)
        short = np.nonzero(lens <= LONG_SEGMENT)[0]
        chunks, carry = [], []
        for i in np.nonzero(lens > LONG_SEGMENT)[0]:
            first, count = int(segments.first[i]), int(lens[i])
            carry.append((int(segments.rows[i]), len(chunks), -(-count // CHUNK)))
            chunks += [(first + off, min(CHUNK, count - off), len(chunks) + off // CHUNK) for off in range(0, count, CHUNK)]
        chunks = np.array(chunks, dtype=np.int64).reshape(-1, 3)
        return dict(short_start=segments.first[short], short_len=lens[short], short_row=np.asarray(segments.rows)[short],
                    chunk_start=chunks[:, 0], chunk_len=chunks[:, 1], chunk_index=chunks[:, 2],
                    carry=np.array(carry, dtype=np.int64).reshape(-1))

    def refresh_single_tokens(self, arrays, segments):
        return True         # single tokens in the same rows: nothing here depends on their positions


_PLANNER = ScanPlanner()


class GatedLinearAttention(Mixer):
    """names: dict with keys q, k, v, g, o, a1, a2 (projection names) and norm (the output norm's weight).
    ``suffixes``: what the checkpoint appends to a projection's name for weight and bias."""
    graph_safe = True

    def __init__(self, hidden_size, n_heads, key_dim, value_dim, decay_rank, *, tau, norm_eps, names,
                 q_scale=None, suffixes=(".weight", ".bias"), norm_suffix=".weight"):
        self.hidden_size, self.n_heads = int(hidden_size), int(n_heads)
        self.key_dim, self.value_dim, self.decay_rank = int(key_dim), int(value_dim), int(decay_rank)
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        if not self.tau > 0:
            raise ValueError("tau must be positive")
        self.q_scale = float(q_scale) if q_scale is not None else self.key_dim ** -0.5
        kw, vw = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        self.projection = StackedLinear(hidden_size, [(names["q"], kw), (names["k"], kw), (names["v"], vw),
                                                      (names["g"], vw), (names["a1"], self.decay_rank)],
                                        suffixes=suffixes)
        self.columns = (0, kw, 2 * kw, 2 * kw + vw, 2 * kw + 2 * vw)
        self.decay_up = Param((kw, self.decay_rank), std=0.2)
        self.decay_bias = Param((kw,), init="zeros")
        self.norm_weight = Param((self.value_dim,), init="norm", std=0.05)
        self._names = {names["a2"] + suffixes[0]: self.decay_up, names["a2"] + suffixes[1]: self.decay_bias,
                       names["norm"] + norm_suffix: self.norm_weight}
        self.out = Linear(vw, hidden_size, name=names["o"], suffixes=suffixes)
        self._needs_scratch = False

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.projection, self.out]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        common = self.projection._weight().dtype
        for param in (self.decay_up, self.decay_bias, self.norm_weight):
            param.data = param.data.to(common).contiguous()
        self._needs_scratch = ops.gla_scan_needs_scratch(self.key_dim, self.value_dim)

    def cache_spec(self):
        return StateSpec((self.n_heads, self.key_dim, self.value_dim), torch.float32)

    def step_planners(self):
        return {**super().step_planners(), _PLANNER.key: _PLANNER}

    takes_norm = True

    def forward(self, ctx, x, cache, residual=None, norm=None):
        """x [N, hidden] -> [N, hidden] (+ residual); ``cache`` is a StateView with one slot per request row."""
        projected = self.projection.forward(ctx, x, norm=norm)
        mixed = ctx.empty((x.shape[0], self.n_heads * self.value_dim))
        self.scan(ctx, projected, cache, mixed)
        return self.out.forward(ctx, mixed, residual=residual)

    def scan(self, ctx, projected, cache, mixed):
        """The recurrence, the norm and the gate over the step's segments: ``projected`` -> ``mixed``."""
        n = projected.shape[0]
        plan = ctx.plans[_PLANNER.key]
        scratch = ctx.empty((n, self.n_heads * self.value_dim), dtype=torch.float32) if self._needs_scratch else None
        alpha = ops.gla_decay(projected, self.columns[4], self.decay_up.data, self.decay_bias.data, self.tau)
        common = (projected, self.columns, alpha, self.q_scale, self.norm_weight.data, self.norm_eps)
        sizes = (self.n_heads, self.key_dim, self.value_dim, mixed)
        n_short, n_chunks = plan.count["short_start"], plan.count["chunk_start"]
        if n_short:
            ops.gla_scan(*common, cache.slots, plan.array["short_start"], plan.array["short_len"],
                         plan.array["short_row"], n_short, *sizes, scratch=scratch)
        if n_chunks:
            chunk = (plan.array["chunk_start"], plan.array["chunk_len"], plan.array["chunk_index"], n_chunks)
            states = ctx.empty((n_chunks, self.n_heads, self.key_dim, self.value_dim), dtype=torch.float32)
            decays = ctx.empty((n_chunks, self.n_heads, self.key_dim), dtype=torch.float32)
            ops.gla_scan(*common, states, *chunk, *sizes, mode=ops.GLA_OWN_STATE, decay_product=decays)
            ops.gla_carry(states, decays, cache.slots, plan.array["carry"], plan.count["carry"] // 3)
            ops.gla_scan(*common, states, *chunk, *sizes, scratch=scratch, mode=ops.GLA_FROM_STATE)
        if scratch is not None:
            ops.gla_norm_gate(scratch, projected, self.columns[3], self.norm_weight.data, self.norm_eps, self.n_heads,
                              self.value_dim, mixed)
        return mixed


class DecayLinearAttention(Mixer):
    """Linear attention with one fixed decay per head (a state matrix per head and request, float32):

        q_t = silu(Wq x_t), k_t = silu(Wk x_t)  [H][d];   v_t = silu(Wv x_t)  [H][e]
        S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t                   S_0 = 0
        y_t = Wo ( o_t / sqrt(mean(o_t^2) + eps) * w  *  sigmoid(Wg x_t) )     one norm over all heads' H * e values

    q, k, v and the gate are one stacked product.  The recurrence is the scan of :class:`GatedLinearAttention`
    (``kernels.ops.gla_scan``) with a decay per head in place of decays per token and the activation applied as
    q, k and v are read; it shares that mixer's step plan, so short segments run token by token and long ones as
    chunks with a carry.  The scan leaves the un-normed outputs in float32; ``kernels.ops.lin_norm_gate_whole``
    norms a token's whole row and gates it.

    names: dict with keys q, k, v, g, o (projection names) and norm (the output norm's weight)."""
    graph_safe = True

    def __init__(self, hidden_size, n_heads, key_dim, value_dim, decay, *, norm_eps, names,
                 suffixes=(".weight", ".bias"), norm_suffix=".weight"):
        self.hidden_size, self.n_heads = int(hidden_size), int(n_heads)
        self.key_dim, self.value_dim, self.norm_eps = int(key_dim), int(value_dim), float(norm_eps)
        self.decay = [float(v) for v in decay]
        if len(self.decay) != self.n_heads or any(not 0.0 <= v <= 1.0 for v in self.decay):
            raise ValueError("one decay in [0, 1] per head")
        kw, vw = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        self.projection = StackedLinear(hidden_size, [(names["q"], kw), (names["k"], kw), (names["v"], vw), (names["g"], vw)],
                                        suffixes=suffixes)
        self.columns = (0, kw, 2 * kw, 2 * kw + vw)
        self.norm_weight = Param((vw,), init="norm", std=0.05)
        self._names = {names["norm"] + norm_suffix: self.norm_weight}
        self.out = Linear(vw, hidden_size, name=names["o"], suffixes=suffixes)
        self._decay = None

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.projection, self.out]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        self.norm_weight.data = self.norm_weight.data.to(self.projection._weight().dtype).contiguous()
        self._decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        ops.gla_scan_needs_scratch(self.key_dim, self.value_dim)       # refuses key sizes the scan cannot hold

    def cache_spec(self):
        return StateSpec((self.n_heads, self.key_dim, self.value_dim), torch.float32)

    def step_planners(self):
        return {**super().step_planners(), _PLANNER.key: _PLANNER}

    def forward(self, ctx, x, cache, residual=None, out_float32=False):
        """x [N, hidden] -> [N, hidden] (+ residual); ``cache`` is a StateView with one slot per request row."""
        projected = self.projection.forward(ctx, x)
        raw = self.scan(ctx, projected, cache)
        mixed = ctx.empty((x.shape[0], self.n_heads * self.value_dim))
        ops.lin_norm_gate_whole(raw, projected, self.columns[3], self.norm_weight.data, self.norm_eps, mixed)
        return self.out.forward(ctx, mixed, residual=residual, out_float32=out_float32)

    def scan(self, ctx, projected, cache):
        """The recurrence over the step's segments: ``projected`` -> the un-normed outputs, float32 [N, heads * e]."""
        n, heads, d, e = projected.shape[0], self.n_heads, self.key_dim, self.value_dim
        plan = ctx.plans[_PLANNER.key]
        raw = ctx.empty((n, heads * e), dtype=torch.float32)
        common = (projected, self.columns, None, 1.0, None, self.norm_eps)
        options = dict(head_decay=self._decay, silu_inputs=True, raw_only=True)
        n_short, n_chunks = plan.count["short_start"], plan.count["chunk_start"]
        if n_short:
            ops.gla_scan(*common, cache.slots, plan.array["short_start"], plan.array["short_len"], plan.array["short_row"],
                         n_short, heads, d, e, None, scratch=raw, **options)
        if n_chunks:
            chunk = (plan.array["chunk_start"], plan.array["chunk_len"], plan.array["chunk_index"], n_chunks)
            states = ctx.empty((n_chunks, heads, d, e), dtype=torch.float32)
            decays = ctx.empty((n_chunks, heads, d), dtype=torch.float32)
            ops.gla_scan(*common, states, *chunk, heads, d, e, None, mode=ops.GLA_OWN_STATE, decay_product=decays, **options)
            ops.gla_carry(states, decays, cache.slots, plan.array["carry"], plan.count["carry"] // 3)
            ops.gla_scan(*common, states, *chunk, heads, d, e, None, scratch=raw, mode=ops.GLA_FROM_STATE, **options)
        return raw
