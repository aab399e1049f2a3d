"""Larolorn written plainly: one function per mechanism, whole sequences, no cache, no batching.

A slow restatement of the design's equations for the tests to compare the engine with.  It shares no
code with the engine: weights come as a dict of checkpoint name -> CPU tensor, the configuration as the
dict that config.json holds.  ``dtype`` is the arithmetic's precision (float32 or float64); the
bfloat16 yardstick (``low``) rounds the outputs of projections and activations, and nothing of what the
design computes in 32 bits (angles, scores, softmax, norms, the recurrent state, the residual sum).

Notation: T tokens at positions t = 0..T-1, width W, H query heads, G key/value heads, d the size of a
query or key head, e the size of a value head, r the rotated dimensions, c the size of the latent, C the
size of a window or a chunk.
"""
from __future__ import annotations

import math

import torch


def _round(x, low):
    return x if low is None else x.to(low).to(x.dtype)


def linear(x, weight, bias=None, low=None):
    """y = x W^T (+ b), W stored [out, in]; input and result rounded when the arithmetic is low precision."""
    y = _round(x, low) @ weight.to(x.dtype).t()
    if bias is not None:
        y = y + bias.to(x.dtype)
    return _round(y, low)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


def angles(T, rot, dtype):
    """a[t, i] = t * base^(-2 i / dims) for i < dims / 2, in float32 like the design's positions (float64 when asked)."""
    dims, base = rot["dims"], rot["base"]
    kind = torch.float64 if dtype == torch.float64 else torch.float32
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64).to(kind)
    return torch.arange(T, dtype=kind)[:, None] * f[None, :]


def rotate_interleaved(x, rot):
    """x [T, ..., n]: the first dims entries are pairs (2 i, 2 i + 1), each turned by the angle of its position."""
    dims = rot["dims"]
    a = angles(x.shape[0], rot, x.dtype).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = a.cos().view(shape), a.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_halves(x, rot):
    """x [T, ..., n]: of the first dims entries, entry i pairs with entry i + dims / 2."""
    dims = rot["dims"]
    half = dims // 2
    a = angles(x.shape[0], rot, x.dtype).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = a.cos().view(shape), a.sin().view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def window_softmax_attention(q, k, v, scale, window):
    """q [T, H, n], k [T, H, n], v [T, H, e] -> [T, H, e]: position i sees i - window < j <= i, plain softmax."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        first = max(0, i - window + 1)
        for h in range(H):
            p = torch.softmax((k[first:i + 1, h] @ q[i, h]) * scale, dim=0)
            out[i, h] = p @ v[first:i + 1, h]
    return out


def latent_attention_mixer(h, w, prefix, m, eps, low=None):
    """Keys and values grow out of one small latent per token; one rotated key part is shared by the heads.

    q_t = Wq h_t, per head [d plain, r rotated];  (l_t, s_t) = Wdkv h_t with c and r rows;
    z_t = rms_norm(l_t) * w;  key of head a = [Wuk_a z_t, rot(s_t)], value = Wuv_a z_t;
    the head's output times sigmoid(Wg h_t)_a; then Wo."""
    T = h.shape[0]
    H, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = linear(h, w[prefix + "q"], low=low).view(T, H, d + r)
    down = linear(h, w[prefix + "dkv"], low=low)
    latent = _round(rms_norm(down[:, :c], w[prefix + "dkv.norm"], eps), low)
    shared = _round(rotate_interleaved(down[:, c:], m["rot"]), low)
    q_plain, q_turned = q[..., :d], _round(rotate_interleaved(q[..., d:].contiguous(), m["rot"]), low)
    k_plain = linear(latent, w[prefix + "uk"], low=low).view(T, H, d)
    value = linear(latent, w[prefix + "uv"], low=low).view(T, H, e)
    keys = torch.cat([k_plain, shared[:, None, :].expand(T, H, r)], dim=-1)
    queries = torch.cat([q_plain, q_turned], dim=-1)
    mixed = window_softmax_attention(queries, keys, value, m["scale"], m["mask"]["size"])
    gate = torch.sigmoid(linear(h, w[prefix + "g"], low=low))
    mixed = _round(mixed * gate[:, :, None], low)
    return linear(mixed.reshape(T, H * e), w[prefix + "o"], low=low)


def sink_softmax(scores, sink):
    """p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)): the sink has no key and no value and counts once."""
    peak = torch.maximum(scores.max(), sink)
    e = torch.exp(scores - peak)
    return e / (torch.exp(sink - peak) + e.sum())


def chunk_sink_attention(q, k, v, scale, chunk, sinks):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e]: position i sees the j <= i of its own chunk
    (floor(i / C) = floor(j / C)); head a reads key/value head floor(a / (H / G)); softmax with the head's sink."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        first = (i // chunk) * chunk
        for a in range(H):
            g = a // (H // G)
            p = sink_softmax((k[first:i + 1, g] @ q[i, a]) * scale, sinks[a].to(q.dtype))
            out[i, a] = p @ v[first:i + 1, g]
    return out


def chunk_attention_mixer(h, w, prefix, m, eps, low=None):
    """Biased projections; q and k are each normed over the whole projection, then turned by halves, then the
    chunked attention with sinks and the biased output product."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w[prefix + "q"], w[prefix + "q.b"], low)
    k = linear(h, w[prefix + "k"], w[prefix + "k.b"], low)
    v = linear(h, w[prefix + "v"], w[prefix + "v.b"], low).view(T, G, e)
    q = rotate_halves(rms_norm(q, w[prefix + "q.norm"], eps).view(T, H, d), m["rot"])
    k = rotate_halves(rms_norm(k, w[prefix + "k.norm"], eps).view(T, G, d), m["rot"])
    mixed = chunk_sink_attention(_round(q, low), _round(k, low), v, m["scale"], m["mask"]["size"], w[prefix + "sink"])
    return linear(_round(mixed.reshape(T, H * e), low), w[prefix + "o"], w[prefix + "o.b"], low)


def silu(z):
    return z * torch.sigmoid(z)


def decayed_state_scan(q, k, v, decay, state=None):
    """q, k [T, H, d], v [T, H, e]: S_t = decay_a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; returns (o [T, H, e], S)."""
    T, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=q.dtype) if state is None else state.clone()
    rate = torch.tensor(decay, dtype=q.dtype).view(H, 1, 1)
    out = torch.zeros(T, H, e, dtype=q.dtype)
    for t in range(T):
        S = rate * S + k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out, S


def decay_mixer(h, w, prefix, m, eps, low=None):
    """silu on the q, k, v projections, the decayed state, one norm over all heads' outputs, a sigmoid gate, Wo."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = _round(silu(linear(h, w[prefix + "q"], low=low)), low).view(T, H, d)
    k = _round(silu(linear(h, w[prefix + "k"], low=low)), low).view(T, H, d)
    v = _round(silu(linear(h, w[prefix + "v"], low=low)), low).view(T, H, e)
    o, _ = decayed_state_scan(q, k, v, m["decay"])
    o = rms_norm(o.reshape(T, H * e), w[prefix + "norm"], eps) * torch.sigmoid(linear(h, w[prefix + "g"], low=low))
    return linear(_round(o, low), w[prefix + "o"], low=low)


def parallel_mixer(h, w, prefix, m, eps, low=None):
    """Half the sum of the two mixers' outputs, each normed over the width with a weight of its own."""
    left = chunk_attention_mixer(h, w, prefix + "left.", m["left"], eps, low)
    right = decay_mixer(h, w, prefix + "right.", m["right"], eps, low)
    return 0.5 * (rms_norm(left, w[prefix + "left.out"], eps) + rms_norm(right, w[prefix + "right.out"], eps))


SWISH_ALPHA = 1.702


def clamped_feed_forward(h, w, prefix, mlp, low=None):
    """g = min(gate h, L), u = clamp(up h, -L, L); down(g sigmoid(1.702 g) (u + 1))."""
    limit = mlp["limit"]
    g = torch.clamp(linear(h, w[prefix + "gate"], low=low), max=limit)
    u = torch.clamp(linear(h, w[prefix + "up"], low=low), min=-limit, max=limit)
    return linear(_round(g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1.0), low), w[prefix + "down"], low=low)


def forward(config, w, tokens, dtype=torch.float64, low=None, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer run)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = w["embed"][tokens].to(dtype)
    after = []
    for i, layer in enumerate(config["layers"]):
        source = layer.get("weights_of")
        p = f"l{i if source is None else source}."
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            y = latent_attention_mixer(x, w, p + "mix.", m, eps, low)
        else:
            y = parallel_mixer(x, w, p + "mix.", m, eps, low)
        x = x + mult * rms_norm(y, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            x = x + mult * rms_norm(clamped_feed_forward(x, w, p + "mlp.", mlp, low), w[p + "norm2"], eps)
        after.append(x.clone())
    h = rms_norm(x, w["final.norm"], eps)
    logits = (_round(h, low) @ w["head"].to(dtype).t()) * config["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits
