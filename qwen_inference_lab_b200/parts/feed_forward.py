"""Feed-forwards: the gated ``down(silu(gate(x)) * up(x))`` (qil/model.py:38-40,70-71) and the plain
``down(act(up(x)))`` of designs without a gate matrix (:class:`PlainMLP`).

gate and up are one stacked product; the activation rounds ``silu(gate)`` to the
activation dtype before the multiply, as elementwise tensor code does.  In
bfloat16 the product and the activation are one kernel: the weight-streaming
kernel for a decode step's few rows, the tcgen05 kernel for prompt portions.

Other activations (``activation``: ``gelu_tanh``, or ``clamped_swish`` with ``limit`` and ``alpha``, see
``kernels.ops.gated_activation``) and biases on the three projections take the stacked product and an
activation kernel of their own.
"""
from __future__ import annotations

import torch

from ..kernels import gemm_tc, ops
from .base import FeedForward
from .linear import Linear, StackedLinear


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size, intermediate_size, *, names, activation="silu", limit=0.0, alpha=1.0, bias=False,
                 suffixes=(".weight", ".bias")):
        """names: dict with keys gate, up, down (projection names without ``.weight``)."""
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (known: {sorted(ops.ACTIVATIONS)})")
        self.activation, self.limit, self.alpha, self.bias = activation, float(limit), float(alpha), bool(bias)
        self.gate_up = StackedLinear(hidden_size, [(names["gate"], intermediate_size),
                                                   (names["up"], intermediate_size)], bias=bias, suffixes=suffixes)
        self.down = Linear(intermediate_size, hidden_size, name=names["down"], bias=bias, suffixes=suffixes)

        self.pairs8 = False

    def children(self):
        return [self.gate_up, self.down]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        w = self.gate_up._w
        inner = self.intermediate_size
        if w.dtype == torch.bfloat16 and inner % 8 == 0 and self.hidden_size % 8 == 0 \
                and self.activation == "silu" and not self.bias:
            # rows as groups of [8 gate, 8 up]: a block of the decode GEMM then holds matching gate and up
            # features and applies the activation in its epilogue
            self.gate_up._w = w.view(2, inner // 8, 8, self.hidden_size).transpose(0, 1).reshape(
                2 * inner, self.hidden_size).contiguous()
            self.pairs8 = True

    takes_norm = True

    def forward(self, ctx, x, residual=None, norm=None, out_float32=False):
        """With ``norm`` x is the block's un-normed input; a decode step's few rows get the norm inside
        the gate/up kernel, longer steps a norm kernel of their own.  ``out_float32``: the down product's float32
        sums are returned as they are (for a block that norms the branch before it joins the stream)."""
        if self.activation != "silu" or self.bias or out_float32:
            gate_up = self.gate_up.forward(ctx, x, norm=norm)
            hidden = ops.gated_activation(gate_up, self.activation, limit=self.limit, alpha=self.alpha, pairs8=self.pairs8)
            return self.down.forward(ctx, hidden, residual=residual, out_float32=out_float32)
        rms = norm.as_rms() if norm is not None else None
        if self.pairs8 and ops.small_m_ok(x, self.gate_up._w) and rms is not None and rms[0].dtype == torch.bfloat16:
            hidden = ops.gemm_small_m(x, self.gate_up._w, silu_pairs=True, norm_weight=rms[0], norm_eps=rms[1])
            return self.down.forward(ctx, hidden, residual=residual)
        if norm is not None:
            x = norm.forward(ctx, x)
        if self.pairs8 and ops.small_m_ok(x, self.gate_up._w):
            hidden = ops.gemm_small_m(x, self.gate_up._w, silu_pairs=True)
        elif self.pairs8 and gemm_tc.usable(x, self.gate_up._w):
            # prompt portions: the tcgen05 kernel applies the activation in its epilogue, so the
            # [tokens, 2 * intermediate] product never goes to memory
            hidden = gemm_tc.gemm_tc(x, self.gate_up._w, silu_pairs=True)
        else:
            gate_up = self.gate_up.forward(ctx, x)
            hidden = ops.silu_mul(gate_up, pairs8=self.pairs8)
        return self.down.forward(ctx, hidden, residual=residual)


class PlainMLP(FeedForward):
    """``down(act(up x))`` without a gate matrix; ``activation`` is one of ``ops.PLAIN_ACTIVATIONS`` (``relu2``: the
    square of relu).  names: dict with keys up, down.  The up product, an activation kernel, the down product
    (with the residual, and a learned scale per feature on the way into it, in its last kernel)."""
    graph_safe = True
    takes_norm = True
    takes_out_scale = True

    def __init__(self, hidden_size, intermediate_size, *, names, activation="relu2", bias=False,
                 suffixes=(".weight", ".bias")):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation not in ops.PLAIN_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (known: {ops.PLAIN_ACTIVATIONS})")
        self.activation = activation
        self.up = Linear(hidden_size, intermediate_size, name=names["up"], bias=bias, suffixes=suffixes)
        self.down = Linear(intermediate_size, hidden_size, name=names["down"], bias=bias, suffixes=suffixes)

    def children(self):
        return [self.up, self.down]

    def forward(self, ctx, x, residual=None, norm=None, out_scale=None, out_float32=False):
        hidden = self.up.forward(ctx, x, norm=norm, activation=self.activation)
        return self.down.forward(ctx, hidden, residual=residual, out_scale=out_scale, out_float32=out_float32)
