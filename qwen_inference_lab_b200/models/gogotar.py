"""Gogotar as an arrangement of parts, with the checkpoint's tensor names.

Layer i (tensors ``l<i>.*``) norms on both sides of each sublayer, with layer norms that have a weight and no bias:
x <- x + norm1b(mixer(norm1 x)), x <- x + norm2b(ff(norm2 x)).  ``loop`` runs layers start .. stop - 1 several times in
a row with the same tensors; every run keeps a cache of its own (one more call of the same block in the decoder's
order).  A token's row of ``embed`` enters the stream times ``embedding.scale``; after ``final.norm`` the same table is
the head, and the logits are capped: cap * tanh(logits / cap).  The residual stream, the norms, the angles of the
rotation, attention scores and the routers are float32 whatever the activation dtype is.

``attention``         a grouped attention without a value projection: a position's value is its key as projected.
                      q and k are normed per head (one weight of ``dim`` for all heads), rotated by halves over the
                      first ``rot.dims`` dimensions with frequencies that ``rot.scaling`` stretches; capped scores
                      inside chunks of ``mask.size`` positions, a learned sink per head, a sigmoid gate per head.
``latent_attention``  queries through a normed latent of their own, keys and values out of one normed latent per
                      token, which is all the cache keeps (``parts.latent_attention``); causal, a learned sink per
                      head, a sigmoid gate per output element; no positions.
``dense``             down(g * sigmoid(1.702 g) * (u + 1)), g = min(gate x, limit), u = clamp(up x, -limit, limit).
``moe``               softmax over all experts' router logits, the ``top`` largest scores weigh their experts
                      unrenormalised; an expert is down(silu(gate x) * up x).
"""
from __future__ import annotations

import torch

from ..config.model_config import GogotarConfig
from ..config.registry import register
from ..parts import (DecoderModel, GatedMLP, GroupedQueryAttention, LatentAttention, LayerCall, LayerNorm, Linear,
                     RotaryFrequencies, RoutedExperts, SandwichNormBlock, TokenEmbedding)

BARE = ("", ".b")          # this design's tensors carry the projection's own name
SWISH_ALPHA = 1.702        # the dense feed-forward's activation: g * sigmoid(1.702 g)


def _attention(width, m, prefix, eps):
    rot = m["rot"]
    scaling = rot.get("scaling")
    position = RotaryFrequencies(rot["dims"], rot["base"], "halves",
                                 scaling=None if scaling is None else (scaling["factor"], scaling["low"],
                                                                       scaling["high"], scaling["original"]))
    names = {k: prefix + k for k in ("q", "k", "o", "sink")}
    names.update(q_norm=prefix + "q.norm", k_norm=prefix + "k.norm")
    return GroupedQueryAttention(width, m["heads"], m["kv_heads"], m["dim"], names=names, scale=m["scale"],
                                 suffixes=BARE, position=position, qk_norm_eps=eps, norm_suffix="",
                                 chunk=(m.get("mask") or {}).get("size", 0), softcap=m.get("softcap") or 0.0,
                                 sink="learned", values_from_keys=True, head_gate=prefix + "g")


def _latent(width, m, prefix, eps):
    names = {k: prefix + k for k in ("dq", "uq", "dkv", "uk", "uv", "g", "o", "sink")}
    names.update(dq_norm=prefix + "dq.norm", dkv_norm=prefix + "dkv.norm")
    return LatentAttention(width, m["heads"], m["dim"], 0, m["vdim"], m["kv_rank"], scale=m["scale"], window=0,
                           position=None, norm_eps=eps, names=names, suffixes=BARE, norm_suffix="",
                           query_latent=m["q_rank"], sink="learned", gate="element")


def _feed_forward(width, mlp, prefix):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return GatedMLP(width, mlp["ff"], names={k: prefix + k for k in ("gate", "up", "down")},
                        activation="clamped_swish", limit=mlp["limit"], alpha=SWISH_ALPHA, suffixes=BARE)
    names = dict(router=prefix + "router", router_bias=None, expert=lambda index, which: f"{prefix}e{index}.{which}")
    return RoutedExperts(width, mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"], names=names,
                         activation="silu", routing="softmax_all", renormalize=False)


def build_gogotar(config: GogotarConfig) -> DecoderModel:
    width, eps = config.width, config.eps
    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        build = _latent if layer["type"] == "latent_attention" else _attention
        layers.append(SandwichNormBlock(width, eps, build(width, layer["mixer"], prefix + "mix.", eps),
                                        _feed_forward(width, layer.get("mlp"), prefix + "mlp."), kind="layer",
                                        names=tuple(prefix + k for k in ("norm1", "norm1b", "norm2", "norm2b")),
                                        norm_suffix=""))
    embedding = TokenEmbedding(config.vocab_size, width, name="embed", suffix="", scale=config.embedding_scale)
    return DecoderModel(config=config, embedding=embedding, layers=layers,
                        order=[LayerCall(i) for i in config.layer_runs()],
                        final_norm=LayerNorm(width, eps, name="final.norm", suffixes=("", ".b"), bias=False),
                        head=Linear(width, config.vocab_size, name="embed", weight=embedding.weight, suffixes=BARE),
                        max_positions=config.max_positions, stream_dtype=torch.float32,
                        logit_softcap=config.logit_softcap)


ARCHITECTURE = register(GogotarConfig.architecture, GogotarConfig.model_type, GogotarConfig, build_gogotar)
