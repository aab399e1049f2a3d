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
:class:`SandwichNormBlock` norms on both sides of each sublayer: x <- x + post1(mixer(pre1 x)), x <- x + post2(ff(pre2 x)).
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


class SandwichNormBlock(Part):
    """x <- x + post1(mixer(pre1(x))), then x <- x + post2(ff(pre2(x))): a norm in front of each sublayer and one on its
    output before it joins the stream, all four of one ``kind`` (``"layer"``: the layer norm without a bias, or
    ``"rms"``) with a weight each, float32 arithmetic.  The sublayers give float32 rows; ``ops.norm_join`` norms a
    branch, adds it to the stream and, in the same kernel, norms the new stream for the sublayer that reads it next.
    That also holds from block to block: a block leaves its feed-forward's branch unjoined in
    ``ctx.extras["pending_join"]`` and the next block of this kind joins it together with its own first norm; the
    decoder settles what is left before anyone else reads the stream (:func:`settle_stream`).
    ``feed_forward`` may be None; the second pair of weights is then optional.
    names: the four weights' names (pre1, post1, pre2, post2)."""
    takes_pending_join = True

    def __init__(self, width, eps, mixer, feed_forward, *, names, kind="layer", norm_suffix=".weight"):
        if kind not in ops.NORM_KINDS:
            raise ValueError(f"unknown norm {kind!r} (known: {sorted(ops.NORM_KINDS)})")
        self.width, self.eps, self.kind = int(width), float(eps), kind
        self.mixer, self.feed_forward = mixer, feed_forward
        optional = feed_forward is None
        self.pre1, self.post1 = Param((width,), init="norm", std=0.05), Param((width,), init="norm", std=0.05)
        self.pre2 = Param((width,), init="norm", std=0.05, optional=optional)
        self.post2 = Param((width,), init="norm", std=0.05, optional=optional)
        self._names = {name + norm_suffix: param for name, param in zip(names, (self.pre1, self.post1, self.pre2, self.post2))}
        if len(names) != 4 or len(self._names) != 4:
            raise ValueError("a block with norms on both sides of its sublayers has four norm weights")
        self.graph_safe = True

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [part for part in (self.mixer, self.feed_forward) if part is not None]

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        weights = [p for p in (self.pre1, self.post1, self.pre2, self.post2) if p.data is not None]
        if len({p.data.dtype for p in weights}) > 1:       # one kernel reads two of them: one dtype for all
            for p in weights:
                p.data = p.data.float()

    def cache_spec(self):
        return self.mixer.cache_spec()

    def _normed(self, ctx, x, weight):
        if self.kind == "layer":
            return ops.layernorm_exact(x, weight, None, self.eps, out_dtype=ctx.dtype)
        return ops.rmsnorm_exact(x, weight, self.eps, out_dtype=ctx.dtype)

    def forward(self, ctx, x, cache):
        """x [N, width] is the residual stream; updated in place and returned."""
        pending = ctx.extras.pop("pending_join", None)
        if pending is not None and pending.stream is x and pending.weight.dtype == self.pre1.data.dtype:
            rows = ctx.empty(x.shape)
            ops.norm_join(x, pending.branch, pending.weight, pending.eps, pending.kind, next_weight=self.pre1.data,
                          next_eps=self.eps, next_kind=self.kind, rows=rows)
        else:
            if pending is not None:
                pending.settle()
            rows = self._normed(ctx, x, self.pre1.data)
        branch = self.mixer.forward(ctx, rows, cache, out_float32=True)
        if self.feed_forward is None:
            ctx.extras["pending_join"] = PendingJoin(x, branch, self.post1.data, self.eps, self.kind)
            return x
        rows = ctx.empty(x.shape)
        ops.norm_join(x, branch, self.post1.data, self.eps, self.kind, next_weight=self.pre2.data, rows=rows)
        branch = self.feed_forward.forward(ctx, rows, out_float32=True)
        ctx.extras["pending_join"] = PendingJoin(x, branch, self.post2.data, self.eps, self.kind)
        return x


class PendingJoin:
    """A normed branch that has not joined its stream yet: stream += norm(branch) * weight."""
    __slots__ = ("stream", "branch", "weight", "eps", "kind")

    def __init__(self, stream, branch, weight, eps, kind):
        self.stream, self.branch, self.weight, self.eps, self.kind = stream, branch, weight, eps, kind

    def settle(self):
        ops.norm_join(self.stream, self.branch, self.weight, self.eps, self.kind)


def settle_stream(ctx):
    """Join what a block left unjoined (see :class:`SandwichNormBlock`); for whoever reads the stream next."""
    pending = ctx.extras.pop("pending_join", None)
    if pending is not None:
        pending.settle()
