"""Two mixers side by side: both read the same input, each output is normed over the model width with a weight of
its own, and the mixer's result is a weighted sum of the two (half the sum, by default):

    y = share * ( left(h) / rms(left(h)) * w_left + right(h) / rms(right(h)) * w_right )

The two keep their own caches: the mixer's cache spec is the tuple of theirs, its view the tuple of their views.
Inside a block that norms its branches on the way into the stream (:class:`PostNormBlock`) the two norms, the sum,
the block's own norm and the residual sum are one kernel (``kernels.ops.rms_join``), so the mixer joins the stream
itself (``joins_stream``); ``forward`` without a stream returns y in float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, Param


class ParallelMixers(Mixer):
    """``left`` and ``right``: two mixers whose ``forward(ctx, h, cache, out_float32=True)`` gives float32 rows.
    names: dict with keys left_out, right_out (the two output norms' weights)."""
    joins_stream = True

    def __init__(self, hidden_size, left, right, *, norm_eps, names, share=0.5, norm_suffix=".weight"):
        self.hidden_size, self.left, self.right = int(hidden_size), left, right
        self.norm_eps, self.share = float(norm_eps), float(share)
        self.left_weight = Param((hidden_size,), init="norm", std=0.05)
        self.right_weight = Param((hidden_size,), init="norm", std=0.05)
        self._names = {names["left_out"] + norm_suffix: self.left_weight, names["right_out"] + norm_suffix: self.right_weight}
        self.graph_safe = True
        self._counts = tuple(len(spec) if isinstance(spec, tuple) else 1 for spec in (left.cache_spec(), right.cache_spec()))

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.left, self.right]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        if self.left_weight.data.dtype != self.right_weight.data.dtype:
            self.left_weight.data, self.right_weight.data = self.left_weight.data.float(), self.right_weight.data.float()

    def cache_spec(self):
        flat = []
        for spec in (self.left.cache_spec(), self.right.cache_spec()):
            flat.extend(spec if isinstance(spec, tuple) else (spec,))
        return tuple(flat)

    def _views(self, cache):
        n_left = self._counts[0]
        left, right = cache[:n_left], cache[n_left:]
        return (left if n_left > 1 else left[0]), (right if self._counts[1] > 1 else right[0])

    def forward(self, ctx, x, cache, stream=None, norm_weight=None, mult=1.0, out_float32=True, rows=None):
        """x [N, hidden] -> y float32 [N, hidden]; with ``stream`` (the residual stream, updated in place and
        returned): stream += mult * rms(y) * norm_weight, and ``rows`` (bfloat16, optional) receives the stream's
        new values rounded."""
        left_view, right_view = self._views(cache)
        a = self.left.forward(ctx, x, left_view, out_float32=True)
        b = self.right.forward(ctx, x, right_view, out_float32=True)
        if stream is None:
            # y itself: each normed branch times its share, added into zeros
            stream = torch.zeros_like(a)
            for branch, weight in ((a, self.left_weight.data), (b, self.right_weight.data)):
                ops.rms_join(stream, branch, weight, self.norm_eps, self.share)
            return stream
        if norm_weight.dtype != self.left_weight.data.dtype:
            norm_weight = norm_weight.to(self.left_weight.data.dtype)
        return ops.rms_join(stream, a, norm_weight, self.norm_eps, mult, b=b, weight_a=self.left_weight.data,
                            weight_b=self.right_weight.data, pre=self.share, rows=rows)
