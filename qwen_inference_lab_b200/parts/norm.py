"""Norms over the last dimension: root-mean-square norms and a layer norm.

``y = cast(x32 * rsqrt(mean(x32^2) + eps)) * w``: statistics and scaling in float32,
rounded to the activation dtype, then multiplied by the weight (no ``1 + w``), as the
reference's ``ScaleNorm`` does (qil/model.py:15-23).
"""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, Param


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width, eps, *, name):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight = Param((width,), init="norm", std=0.05)

    def named_params(self):
        return {self.name + ".weight": self.weight}

    def forward(self, ctx, x, rows=None):
        """Norm of every row of ``x`` [N, width], or of ``x[rows]`` when ``rows`` (int32) is given."""
        return ops.rmsnorm(x, self.weight.data, self.eps, rows=rows)

    def as_rms(self):
        return self.weight.data, self.eps


class ExactRMSNorm(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * (offset + w)`` with float32 arithmetic and a single rounding.

    ``offset`` 1 is for weights stored around zero.  The input may be a float32 residual stream under
    bfloat16 activations: the result has the activation dtype (``ctx.dtype``).  ``suffix`` is what the
    checkpoint appends to ``name``.
    """
    graph_safe = True

    def __init__(self, width, eps, *, name, offset=0.0, suffix=".weight", optional=False):
        self.width, self.eps, self.offset, self.name, self.suffix = int(width), float(eps), float(offset), name, suffix
        init = ("normal", 0.05) if offset else ("norm", 0.05)
        self.weight = Param((width,), init=init[0], std=init[1], optional=optional)

    def named_params(self):
        return {self.name + self.suffix: self.weight}

    def forward(self, ctx, x, rows=None):
        return ops.rmsnorm_exact(x, self.weight.data, self.eps, self.offset, out_dtype=ctx.dtype, rows=rows)


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * w + b`` with ``var`` the mean of the squared deviations: float32
    arithmetic and a single rounding, like :class:`ExactRMSNorm`, and like it it may read a float32 residual
    stream under bfloat16 activations.  ``suffixes``: what the checkpoint appends to ``name`` for weight and bias.
    ``bias=False``: a layer norm with a weight alone."""
    graph_safe = True

    def __init__(self, width, eps, *, name, suffixes=(".weight", ".bias"), optional=False, bias=True):
        self.width, self.eps, self.name, self.suffixes = int(width), float(eps), name, tuple(suffixes)
        self.weight = Param((width,), init="norm", std=0.05, optional=optional)
        self.bias = Param((width,), init="normal", std=0.05, optional=optional) if bias else None

    def named_params(self):
        params = {self.name + self.suffixes[0]: self.weight}
        if self.bias is not None:
            params[self.name + self.suffixes[1]] = self.bias
        return params

    def finalize(self, device, dtype):
        if self.bias is not None and self.weight.data is not None and self.bias.data.dtype != self.weight.data.dtype:
            self.bias.data = self.bias.data.to(self.weight.data.dtype)

    def forward(self, ctx, x, rows=None):
        return ops.layernorm_exact(x, self.weight.data, self.bias.data if self.bias is not None else None, self.eps,
                                   out_dtype=ctx.dtype, rows=rows)
