"""Mixture of experts: a router picks a few small gated feed-forwards per token.

    logits  = R x + b                              float32
    chosen  = the ``top`` largest logits           (the lower index wins a tie)
    weights = softmax over the chosen logits alone
    y       = sum_chosen weight_e * down_e(act(gate_e x, up_e x))  (+ shared(x), an expert that every token uses)

The experts' matrices are stacked after loading ([experts, ff, width] and [experts, width, ff]); the
tokens are grouped by expert on the device and the products run over the groups
(``kernels.ops.moe_experts``), so nothing about a step's routing reaches the host and a step of single
tokens can be recorded into a CUDA graph.  A token's result is summed in the order of its own choice
and does not depend on the rest of the batch.

Options for other designs of routing:

``routing="softmax_all"``  scores = softmax over all outputs of the router; the choice goes by score + a stored
                           correction (``names["correction"]``), the weights are the chosen scores themselves,
                           divided by their sum (+ 1e-20) and multiplied by ``weight_scale``;
                           ``renormalize=False`` leaves out the division: the chosen scores are the weights
``identity``               so many further outputs of the router, behind the experts', name no expert: a token
                           that chooses one gets weight * x, its own input
``gated=False``            experts without a gate matrix: down_e(act(up_e x)), ``activation`` one without a gate
``shared_gate``            the name of a [1, width] tensor: the shared expert's output is multiplied by
                           sigmoid(gate . x), one number per token (the dot product rides with the router's)
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, Param


class RoutedExperts(FeedForward):
    """names: dict with ``router`` (its weight's full name), ``router_bias`` (or None) and ``expert``: a function
    (index, "gate" | "up" | "down") -> tensor name.  ``activation``: ``clamped_swish`` (with ``limit`` and
    ``alpha``) or ``silu``.  ``shared``: a feed-forward part that runs for every token and is added, or None."""
    graph_safe = True

    def __init__(self, hidden_size, expert_size, n_experts, top, *, names, activation="silu", limit=0.0, alpha=1.0,
                 shared=None, routing="softmax_chosen", weight_scale=1.0, identity=0, gated=True, shared_gate=None,
                 renormalize=True):
        self.hidden_size, self.expert_size = int(hidden_size), int(expert_size)
        self.n_experts, self.top, self.identity = int(n_experts), int(top), int(identity)
        if self.identity < 0 or not 1 <= self.top <= self.n_experts + self.identity:
            raise ValueError(f"{top} of {n_experts} experts (+ {identity} that hand the input through) per token")
        if routing not in ("softmax_chosen", "softmax_all"):
            raise ValueError(f"unknown routing {routing!r}")
        if activation not in (("silu", "clamped_swish") if gated else ops.PLAIN_ACTIVATIONS):
            raise ValueError(f"activation {activation!r} does not fit experts {'with' if gated else 'without'} a gate matrix")
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.routing, self.weight_scale, self.gated = routing, float(weight_scale), bool(gated)
        self.renormalize = bool(renormalize)
        if not self.renormalize and routing != "softmax_all":
            raise ValueError("only the scores of a softmax over all outputs can weigh the experts undivided")
        self.shared = shared
        outputs = self.n_experts + self.identity
        self.router = Param((outputs, hidden_size), std=0.5)
        self.router_bias = Param((outputs,), init="zeros") if names.get("router_bias") else None
        self.correction = Param((outputs,), init="normal", std=0.05) if names.get("correction") else None
        self.shared_gate = Param((1, hidden_size), std=0.1) if shared_gate else None
        if self.shared_gate is not None and (shared is None or self.router_bias is not None):
            raise ValueError("a gate on the shared expert needs that expert, and a router without biases")
        self.gate = [Param((expert_size, hidden_size), std=0.1) for _ in range(n_experts)] if gated else []
        self.up = [Param((expert_size, hidden_size), std=0.1) for _ in range(n_experts)]
        self.down = [Param((hidden_size, expert_size), std=0.1) for _ in range(n_experts)]
        self._names = {names["router"]: self.router}
        if self.router_bias is not None:
            self._names[names["router_bias"]] = self.router_bias
        if self.correction is not None:
            self._names[names["correction"]] = self.correction
        if self.shared_gate is not None:
            self._names[shared_gate] = self.shared_gate
        for index in range(n_experts):
            if gated:
                self._names[names["expert"](index, "gate")] = self.gate[index]
            self._names[names["expert"](index, "up")] = self.up[index]
            self._names[names["expert"](index, "down")] = self.down[index]
        self._gate = self._up = self._down = self._router = None

    def named_params(self):
        return dict(self._names)

    def children(self):
        return [self.shared] if self.shared is not None else []

    def finalize(self, device, dtype):
        super().finalize(device, dtype)
        stack = lambda params: torch.stack([p.data for p in params]).contiguous()
        self._gate = stack(self.gate) if self.gated else None
        self._up, self._down = stack(self.up), stack(self.down)
        for param in (*self.gate, *self.up, *self.down):
            param.data = None
        if self.router_bias is not None:
            self.router_bias.data = self.router_bias.data.to(self.router.data.dtype)
        if self.correction is not None:
            self.correction.data = self.correction.data.to(torch.float32).contiguous()
        self._router = self.router.data
        if self.shared_gate is not None:       # the gate's row behind the router's: one kernel takes all the dot products
            self._router = torch.cat([self.router.data, self.shared_gate.data.to(self.router.data.dtype)]).contiguous()

    takes_out_scale = True

    def forward(self, ctx, x, residual=None, out_scale=None, out_float32=False):
        """``out_float32``: the experts' weighted sum as float32 rows (for a block that norms the branch before it
        joins the stream); without it and without a residual the result has the stream's dtype."""
        if out_float32:
            if residual is not None or out_scale is not None:
                raise ValueError("a float32 result goes without a residual")
            return self._forward_general(ctx, x, None, None, torch.float32)
        if self.routing == "softmax_all" or self.identity or not self.gated or self.shared_gate is not None \
                or out_scale is not None:
            return self._forward_general(ctx, x, residual, out_scale)
        chosen, weights = ops.moe_route(x, self.router.data, self.router_bias.data if self.router_bias else None, self.top)
        out = ops.moe_experts(x, chosen, weights, self._gate, self._up, self._down, self.activation, limit=self.limit,
                              alpha=self.alpha, residual=residual,
                              out=None if residual is not None else ctx.empty(x.shape, dtype=ctx.stream_dtype))
        if self.shared is not None:
            out = self.shared.forward(ctx, x, residual=out)
        return out

    def _forward_general(self, ctx, x, residual, out_scale, out_dtype=None):
        """Every option at once: the shared expert's float32 output, its gate and the output scale go into the
        kernel that sums a token's experts onto the residual."""
        routed = ops.moe_route(x, self._router, self.router_bias.data if self.router_bias else None, self.top,
                               softmax_all=self.routing == "softmax_all",
                               correction=self.correction.data if self.correction is not None else None,
                               weight_scale=self.weight_scale, gate_row=self.shared_gate is not None,
                               renormalize=self.renormalize)
        chosen, weights = routed[:2]
        extra = self.shared.forward(ctx, x, out_float32=True) if self.shared is not None else None
        first, second = (self._gate, self._up) if self.gated else (self._up, None)
        return ops.moe_experts(x, chosen, weights, first, second, self._down, self.activation, limit=self.limit,
                               alpha=self.alpha, residual=residual, identity=self.identity > 0, extra=extra,
                               extra_gate=routed[2] if self.shared_gate is not None else None, col_scale=out_scale,
                               out=None if residual is not None else ctx.empty(x.shape, dtype=out_dtype or ctx.stream_dtype))
