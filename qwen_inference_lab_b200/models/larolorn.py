"""Larolorn as an arrangement of parts, with the checkpoint's tensor names.

Layer i (tensors ``l<i>.*``) reads the residual stream itself and norms each sublayer's output on its way into the
stream: x <- x + m * norm1(mixer(x)), x <- x + m * norm2(ff(x)), m = ``residual_mult``.  A layer with ``weights_of: j``
runs with layer j's tensors and keeps a cache and state of its own.  The residual stream, the norms, the angles of the
rotations, attention scores and the recurrent state are float32 whatever the activation dtype is.

``latent_attention``  keys and values grow out of a small latent per token, which is all the cache keeps
                      (``parts.latent_attention``): interleaved rotation of the rotated part, a sliding window, a
                      sigmoid gate per head on the output.
``parallel``          two mixers side by side (``parts.parallel``), each output normed over the width, half their sum:
                      ``left`` a grouped attention with biased projections, q and k normed over the whole projection,
                      rotation by halves, a chunked mask and a learned sink per head; ``right`` a linear attention
                      with a fixed decay per head (``parts.linear_attention.DecayLinearAttention``).
``dense``             down(g * sigmoid(1.702 g) * (u + 1)), g = min(gate x, limit), u = clamp(up x, -limit, limit).
Then ``final.norm`` and ``head``, whose products are multiplied by ``logit_scale``.
"""
from __future__ import annotations

import torch

from ..config.model_config import LarolornConfig
from ..config.registry import register
from ..parts import (DecayLinearAttention, DecoderModel, ExactRMSNorm, GatedMLP, GroupedQueryAttention, LatentAttention,
                     LayerCall, Linear, ParallelMixers, PostNormBlock, RotaryFrequencies, TokenEmbedding)

BARE = ("", ".b")          # this design's tensors carry the projection's own name; biases add ".b"
SWISH_ALPHA = 1.702        # the feed-forward's activation: g * sigmoid(1.702 g)


def _rotation(rot, layout):
    return RotaryFrequencies(rot["dims"], rot["base"], layout)


def _latent(width, m, prefix, eps):
    names = {k: prefix + k for k in ("q", "dkv", "uk", "uv", "g", "o")}
    names["dkv_norm"] = prefix + "dkv.norm"
    return LatentAttention(width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], scale=m["scale"],
                           window=m["mask"]["size"], position=_rotation(m["rot"], "interleaved"), norm_eps=eps,
                           names=names, suffixes=BARE, norm_suffix="")


def _parallel(width, m, prefix, eps):
    left, right = m["left"], m["right"]
    names = {k: f"{prefix}left.{k}" for k in ("q", "k", "v", "o", "sink")}
    names.update(q_norm=prefix + "left.q.norm", k_norm=prefix + "left.k.norm")
    attention = GroupedQueryAttention(
        width, left["heads"], left["kv_heads"], left["dim"], names=names, bias=True, scale=left["scale"],
        v_head_dim=left["vdim"], suffixes=BARE, position=_rotation(left["rot"], "halves"), chunk=left["mask"]["size"],
        sink="learned", whole_qk_norm_eps=eps, norm_suffix="")
    names = {k: f"{prefix}right.{k}" for k in ("q", "k", "v", "g", "o", "norm")}
    recurrent = DecayLinearAttention(width, right["heads"], right["dim"], right["vdim"], right["decay"], norm_eps=eps,
                                     names=names, suffixes=BARE, norm_suffix="")
    return ParallelMixers(width, attention, recurrent, norm_eps=eps, share=0.5, norm_suffix="",
                          names=dict(left_out=prefix + "left.out", right_out=prefix + "right.out"))


def _feed_forward(width, mlp, prefix):
    if mlp is None:
        return None
    return GatedMLP(width, mlp["ff"], names={k: prefix + k for k in ("gate", "up", "down")}, activation="clamped_swish",
                    limit=mlp["limit"], alpha=SWISH_ALPHA, suffixes=BARE)


def build_larolorn(config: LarolornConfig) -> DecoderModel:
    width, eps = config.width, config.eps
    layers, block_of = [], {}
    for i, layer in enumerate(config.layers):
        if layer.get("weights_of") is None:
            prefix = f"l{i}."
            build = _latent if layer["type"] == "latent_attention" else _parallel
            block_of[i] = len(layers)
            layers.append(PostNormBlock(width, eps, config.residual_mult, build(width, layer["mixer"], prefix + "mix.", eps),
                                        _feed_forward(width, layer.get("mlp"), prefix + "mlp."),
                                        names=(prefix + "norm1", prefix + "norm2"), norm_suffix=""))
    order = [LayerCall(block_of[i if layer.get("weights_of") is None else layer["weights_of"]])
             for i, layer in enumerate(config.layers)]
    return DecoderModel(config=config, embedding=TokenEmbedding(config.vocab_size, width, name="embed", suffix=""),
                        layers=layers, order=order,
                        final_norm=ExactRMSNorm(width, eps, name="final.norm", suffix=""),
                        head=Linear(width, config.vocab_size, name="head", suffixes=BARE),
                        max_positions=config.max_positions, stream_dtype=torch.float32, logit_scale=config.logit_scale)


ARCHITECTURE = register(LarolornConfig.architecture, LarolornConfig.model_type, LarolornConfig, build_larolorn)
