"""Arrangement of a layer's parts: norm -> mixer -> + -> norm -> feed-forward -> +.

The pre-norm order of the reference's ``DecoderBlock.forward`` (qil/model.py:48-71).
The block owns no sizes: it is given a norm, a mixer, a second norm and a
feed-forward, each already built, so different layers of one model may hold
different kinds of each.  ``feed_forward`` may be None: the layer is then its mixer
alone (a second norm given all the same only claims its tensor).

Two options for other designs.  A learned scale per feature on each branch before it joins the stream
(``scales``: the two tensors' names): x <- x + s1 * mixer(norm1 x), x <- x + s2 * ff(norm2 x); a part that sets
``takes_out_scale`` applies the scale in its last kernel, the others' results are scaled and added by a kernel
of the block's.  And parts that run on the stream after the feed-forward (``after``: each ``forward(ctx, x) -> x``).

:class:`PostNormBlock` is the other arrangement: the sublayers read the stream itself and the norm sits on each
sublayer's output, x <- x + m * norm1(mixer(x)), x <- x + m * norm2(ff(x)) with a fixed multiplier m.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Param, Part


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ff_norm, feed_forward, *, scales=None, after=()):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ff_norm, self.feed_forward = ff_norm, feed_forward
        self.after = list(after)
        self.graph_safe = True
        self.mixer_scale = self.ff_scale = None
        self._scale_names = scales
        if scales is not None:
            width = mixer_norm.width
            self.mixer_scale = Param((width,), init="norm", std=0.05)
            self.ff_scale = Param((width,), init="norm", std=0.05, optional=feed_forward is None)

    def named_params(self):
        if self._scale_names is None:
            return {}
        return {self._scale_names[0]: self.mixer_scale, self._scale_names[1]: self.ff_scale}

    def children(self):
        return [part for part in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward, *self.after)
                if part is not None]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        for scale in (self.mixer_scale, self.ff_scale):      # the kernels read the scales as float32
            if scale is not None and scale.data is not None:
                scale.data = scale.data.to(torch.float32).contiguous()

    def _scaled(self, ctx, part, norm, x, scale, *cache):
        """x + scale * part(norm(x)), by the part's own last kernel where it can."""
        if getattr(part, "takes_out_scale", False):
            if getattr(part, "takes_norm", False):
                return part.forward(ctx, x, *cache, residual=x, norm=norm, out_scale=scale)
            return part.forward(ctx, norm.forward(ctx, x), *cache, residual=x, out_scale=scale)
        if getattr(part, "takes_norm", False):
            branch = part.forward(ctx, x, *cache, norm=norm)
        else:
            branch = part.forward(ctx, norm.forward(ctx, x), *cache)
        return ops.scaled_add(x, branch, scale)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        """x [N, hidden] is the residual stream; returned updated (possibly in place)."""
        if self.mixer_scale is not None:
            x = self._scaled(ctx, self.mixer, self.mixer_norm, x, self.mixer_scale.data, cache)
            if self.feed_forward is not None:
                x = self._scaled(ctx, self.feed_forward, self.ff_norm, x, self.ff_scale.data)
            for part in self.after:
                x = part.forward(ctx, x)
            return x
        x = self._plain(ctx, x, cache)
        for part in self.after:
            x = part.forward(ctx, x)
        return x

    def _plain(self, ctx, x, cache):
        if getattr(self.mixer, "takes_norm", False):
            x = self.mixer.forward(ctx, x, cache, residual=x, norm=self.mixer_norm)
        else:
            x = self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), cache, residual=x)
        if self.feed_forward is None:       # a layer without a feed-forward
            return x
        if getattr(self.feed_forward, "takes_norm", False):
            return self.feed_forward.forward(ctx, x, residual=x, norm=self.ff_norm)
        return self.feed_forward.forward(ctx, self.ff_norm.forward(ctx, x), residual=x)


class PostNormBlock(Part):
    """x <- x + mult * rms(mixer(x); w1), then x <- x + mult * rms(ff(x); w2): the sublayers read the residual
    stream itself (cast to the activation dtype when the stream is float32 under bfloat16 activations) and their
    output is normed (root mean square over the width, a weight per feature, float32) before it joins the stream.
    The norm, the multiplier and the sum are one kernel (``kernels.ops.rms_join``), which under bfloat16 activations
    also writes the float32 stream's new values rounded, for the next sublayer to read (the next block finds them
    in ``ctx.extras["stream_rows"]`` as (the stream, its copy); a part that changes the stream between two such blocks
    has to remove that entry), so that only the first block of a step casts the stream.  A mixer that sets
    ``joins_stream`` is handed the stream, the weight and the multiplier and does the join itself (two mixers side
    by side fold their own output norms into that kernel).  ``feed_forward`` may be None; the second norm's weight
    is then optional.  names: (first norm's weight, second norm's weight)."""

    def __init__(self, width, eps, mult, mixer, feed_forward, *, names, norm_suffix=".weight"):
        self.width, self.eps, self.mult = int(width), float(eps), float(mult)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm = Param((width,), init="norm", std=0.05)
        self.ff_norm = Param((width,), init="norm", std=0.05, optional=feed_forward is None)
        self._names = {names[0] + norm_suffix: self.mixer_norm, names[1] + norm_suffix: self.ff_norm}
        self.graph_safe = True

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [part for part in (self.mixer, self.feed_forward) if part is not None]

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        """x [N, width] is the residual stream; updated in place and returned."""
        kept = ctx.extras.pop("stream_rows", None)          # (the stream, its rounded copy) of the block before
        if x.dtype == ctx.dtype:
            rows = x
        else:
            rows = kept[1] if kept is not None and kept[0] is x else ops.cast(x, ctx.dtype)
        copies = x.dtype != ctx.dtype and ctx.dtype == torch.bfloat16
        after = ctx.empty(x.shape) if copies else None
        if getattr(self.mixer, "joins_stream", False):
            x = self.mixer.forward(ctx, rows, cache, stream=x, norm_weight=self.mixer_norm.data, mult=self.mult, rows=after)
        else:
            branch = self.mixer.forward(ctx, rows, cache, out_float32=True)
            x = ops.rms_join(x, branch, self.mixer_norm.data, self.eps, self.mult, rows=after)
        if self.feed_forward is not None:
            rows = x if x.dtype == ctx.dtype else (after if copies else ops.cast(x, ctx.dtype))
            branch = self.feed_forward.forward(ctx, rows, out_float32=True)
            after = ctx.empty(x.shape) if copies else None
            x = ops.rms_join(x, branch, self.ff_norm.data, self.eps, self.mult, rows=after)
        if copies:
            ctx.extras["stream_rows"] = (x, after)
        return x
