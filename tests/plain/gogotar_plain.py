"""Gogotar written plainly: one function per mechanism, whole sequences, no cache, no batching.

A slow restatement of the design's equations for the tests to compare the engine with.  It shares no
code with the engine: weights come as a dict of checkpoint name -> CPU tensor, the configuration as the
dict that config.json holds.  ``dtype`` is the arithmetic's precision (float32 or float64); the
bfloat16 yardstick (``low``) rounds the outputs of projections and activations, and nothing of what the
design computes in 32 bits (angles, scores, softmax, norms, routers, the residual sum).

Notation: T tokens at positions t = 0..T-1, width W, H query heads, G key/value heads, d the size of a
query or key head, e the size of a value head, r the rotated dimensions, c the size of the key/value
latent, C the size of a chunk, E experts of which a token uses K.
"""
from __future__ import annotations

import math

import torch


def _round(x, low):
    return x if low is None else x.to(low).to(x.dtype)


def linear(x, weight, low=None):
    """y = x W^T, W stored [out, in]; input and result rounded when the arithmetic is low precision."""
    return _round(_round(x, low) @ weight.to(x.dtype).t(), low)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w over the last dimension; no bias."""
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(centred.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def scaled_frequencies(rot):
    """f_i = base^(-2 i / r), i < r / 2, then stretched by wavelength l = 2 pi / f as ``rot["scaling"]`` says:
    short waves (l < original / high) stay, long ones (l > original / low) are divided by ``factor``, and between
    the two s = (original / l - low) / (high - low) blends f / factor (s = 0) into f (s = 1).  Python floats."""
    dims, base = rot["dims"], rot["base"]
    result = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if scaling:
        factor, low, high, original = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
        for i, f in enumerate(result):
            wave = 2.0 * math.pi / f
            if wave < original / high:
                continue
            if wave > original / low:
                result[i] = f / factor
            else:
                s = (original / wave - low) / (high - low)
                result[i] = (1.0 - s) * f / factor + s * f
    return result


def rotate_halves(x, rot, first=0):
    """x [T, ..., n]: of the first r entries, entry i pairs with entry i + r / 2; the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i.  ``first``: the position of x[0].  Angles are float32 products of
    float32 positions and frequencies (float64 when the arithmetic is)."""
    dims = rot["dims"]
    half = dims // 2
    kind = torch.float64 if x.dtype == torch.float64 else torch.float32
    f = torch.tensor(scaled_frequencies(rot), dtype=torch.float64).to(kind)
    a = (torch.arange(first, first + x.shape[0], dtype=kind)[:, None] * f[None, :]).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = a.cos().view(shape), a.sin().view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def sink_softmax(scores, sink):
    """p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)): the sink has no key and no value and counts once."""
    peak = torch.maximum(scores.max(), sink)
    e = torch.exp(scores - peak)
    return e / (torch.exp(sink - peak) + e.sum())


def sink_attention(q, k, v, scale, sinks, chunk=0, softcap=0.0):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Position i sees j <= i, with ``chunk`` only the j of its
    own chunk (floor(i / C) = floor(j / C)); head a reads key/value head floor(a / (H / G)); the scaled score is
    capped (cap tanh(score / cap)) when ``softcap`` is set; softmax with the head's sink."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        first = (i // chunk) * chunk if chunk else 0
        for a in range(H):
            g = a // (H // G)
            scores = (k[first:i + 1, g] @ q[i, a]) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            out[i, a] = sink_softmax(scores, sinks[a].to(q.dtype)) @ v[first:i + 1, g]
    return out


def attention_mixer(h, w, prefix, m, eps, low=None):
    """Grouped attention whose values are its keys as projected: q = Wq h, k = Wk h, v = k; q and k are normed per
    head (one weight of d for all heads), turned by halves on their first r dimensions; capped, chunked scores with a
    sink; head a's output times sigmoid(Wg h)_a; Wo."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = linear(h, w[prefix + "q"], low).view(T, H, d)
    k = linear(h, w[prefix + "k"], low).view(T, G, d)
    v = k
    q = rotate_halves(rms_norm(q, w[prefix + "q.norm"], eps), m["rot"])
    k = rotate_halves(rms_norm(k, w[prefix + "k.norm"], eps), m["rot"])
    mask = m.get("mask") or {}
    mixed = sink_attention(_round(q, low), _round(k, low), v, m["scale"], w[prefix + "sink"], mask.get("size", 0),
                           m.get("softcap", 0.0))
    gate = torch.sigmoid(linear(h, w[prefix + "g"], low))                 # [T, H]
    mixed = _round(mixed * gate[:, :, None], low)
    return linear(mixed.reshape(T, H * v.shape[-1]), w[prefix + "o"], low)


def latent_attention_mixer(h, w, prefix, m, eps, low=None):
    """Queries through a normed latent of their own, keys and values out of one normed latent per token:
    c_q = rms(Wdq h) w_q, q = Wuq c_q;  z = rms(Wdkv h) w_z;  head a: k = Wuk_a z, v = Wuv_a z;  causal scores
    (q . k) scale through a softmax with a sink; all heads' outputs times sigmoid(Wg h), element by element; Wo."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q_latent = _round(rms_norm(linear(h, w[prefix + "dq"], low), w[prefix + "dq.norm"], eps), low)
    q = linear(q_latent, w[prefix + "uq"], low).view(T, H, d)
    z = _round(rms_norm(linear(h, w[prefix + "dkv"], low), w[prefix + "dkv.norm"], eps), low)
    k = linear(z, w[prefix + "uk"], low).view(T, H, d)
    v = linear(z, w[prefix + "uv"], low).view(T, H, e)
    mixed = sink_attention(q, k, v, m["scale"], w[prefix + "sink"]).reshape(T, H * e)
    mixed = _round(mixed * torch.sigmoid(linear(h, w[prefix + "g"], low)), low)
    return linear(mixed, w[prefix + "o"], low)


SWISH_ALPHA = 1.702


def clamped_feed_forward(h, w, prefix, mlp, low=None):
    """g = min(gate h, L), u = clamp(up h, -L, L); down(g sigmoid(1.702 g) (u + 1))."""
    limit = mlp["limit"]
    g = torch.clamp(linear(h, w[prefix + "gate"], low), max=limit)
    u = torch.clamp(linear(h, w[prefix + "up"], low), min=-limit, max=limit)
    return linear(_round(g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1.0), low), w[prefix + "down"], low)


def route(h, router, top, low=None):
    """Scores = softmax(R h) over all experts; the ``top`` largest are chosen (the lower index wins a tie) and weigh
    their experts as they are, not renormalised.  Returns (chosen [T, K], weights [T, K])."""
    scores = torch.softmax(_round(h, low) @ router.to(h.dtype).t(), dim=-1)
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(scores, 1, order)


def routed_experts(h, w, prefix, mlp, low=None, margins=None):
    """sum over a token's chosen experts of score_e * down_e(silu(gate_e h) * (up_e h)).  ``margins``: a list that
    receives, per token, by how much of itself the last chosen score leads the first rejected one."""
    top = mlp["router"]["top"]
    chosen, weights = route(h, w[prefix + "router"], top, low)
    if margins is not None and top < mlp["router"]["experts"]:
        ranked = torch.softmax(h @ w[prefix + "router"].to(h.dtype).t(), dim=-1).sort(dim=-1, descending=True).values
        margins.append((ranked[:, top - 1] - ranked[:, top]) / ranked[:, top - 1])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for n in range(top):
            p = f"{prefix}e{int(chosen[t, n])}."
            row = h[t:t + 1]
            gate = linear(row, w[p + "gate"], low)
            hidden = _round(_round(gate * torch.sigmoid(gate), low) * linear(row, w[p + "up"], low), low)
            out[t] += weights[t, n] * linear(hidden, w[p + "down"], low)[0]
    return out


def layer_runs(config):
    """The layers in the order they run: layers start .. stop - 1 of ``loop`` run ``times`` times in a row."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def forward(config, w, tokens, dtype=torch.float64, low=None, return_layers=False, margins=None):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer run).  ``margins``: a list
    that receives every routed layer run's margins (see ``routed_experts``)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = config["norm"]["eps"]
    x = w["embed"][tokens].to(dtype) * config["embedding"]["scale"]
    after = []
    for i in layer_runs(config):
        layer, p = config["layers"][i], f"l{i}."
        mixer = latent_attention_mixer if layer["type"] == "latent_attention" else attention_mixer
        y = mixer(_round(layer_norm(x, w[p + "norm1"], eps), low), w, p + "mix.", layer["mixer"], eps, low)
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            inputs = _round(layer_norm(x, w[p + "norm2"], eps), low)
            if mlp["kind"] == "dense":
                y = clamped_feed_forward(inputs, w, p + "mlp.", mlp, low)
            else:
                y = routed_experts(inputs, w, p + "mlp.", mlp, low, margins)
            x = x + layer_norm(y, w[p + "norm2b"], eps)
        after.append(x.clone())
    h = _round(layer_norm(x, w["final.norm"], eps), low)
    logits = h @ w["embed"].to(dtype).t()
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits
