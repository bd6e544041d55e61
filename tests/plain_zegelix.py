"""A plain, slow implementation of the Zegelix decoder in float64 numpy: one function per mechanism, written from
the design's equations and sharing nothing with the engine.  It runs a whole sequence at once (no cache, no
batching); the engine's tests compare every way of cutting and batching against it.

The design in this file's notation.  T tokens, width D, rms(z) = z / sqrt(mean(z^2) + eps).

* embedding: x_t = E[tok_t] * c_embed; x0 is a copy of it;
* order: ``layers`` lists the layers; the span [loop.start, loop.stop) runs ``loop.times`` times in a row with the same
  weights; right before the first layer of every pass x <- M [x ; x0] (M = ``loop.in``, [D, 2 D]);
* layer: x <- x + mixer(rms(x) w1); x <- x + ff(rms(x) w2) (the feed-forward may be absent);
* mixers: ``gated_linear_recurrence`` (type ``rglru``) and ``pooled_window_attention`` (type ``attention``);
* feed-forward: ``expert_mixture``: routed experts plus a shared expert behind a gate of one number per token;
* output: rms(x) w_final, logits = E x * c_logit (the table without its scale).
"""
from __future__ import annotations

import math

import numpy as np


def rms(z, eps):
    return z / np.sqrt((z * z).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def round_bf16(a):
    """Round float64 values to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


def _same(a):
    return a


# ------------------------------------------------------------------------------------------ recurrence
def causal_conv(u, taps, bias):
    """y[t, c] = bias[c] + sum_j taps[c, j] u[t - (n - 1) + j, c]; inputs before the sequence are zero."""
    T, C = u.shape
    n = taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), u], axis=0)
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for j in range(n):
        y += padded[j:j + T] * taps[:, j]
    return y


def block_gates(u, w, b):
    """sigmoid(w[blk] u_blk + b[blk]) for u cut into len(w) equal parts; w [blocks, out, in]."""
    nb, size = w.shape[0], w.shape[1]
    parts = [u[:, k * size:(k + 1) * size] @ w[k].T + b[k] for k in range(nb)]
    return sigmoid(np.concatenate(parts, axis=1))


def gated_linear_recurrence(h, W, p, m, rounder=_same):
    """Two branches of ``width`` channels: y = gelu_tanh(W_y h + b_y); u = conv(W_x h + b_x); gates r and i from u by
    block-diagonal matrices; log a = -8 r softplus(lam); S_t = a S_(t-1) + sqrt(1 - a^2) i u from S = 0; W_o (S * y)."""
    y = rounder(gelu_tanh(rounder(h @ W[p + "y"].T + W[p + "y.b"])))
    u = rounder(causal_conv(rounder(h @ W[p + "x"].T + W[p + "x.b"]), W[p + "conv"], W[p + "conv.b"]))
    r = block_gates(u, W[p + "ra"], W[p + "ra.b"])
    i = block_gates(u, W[p + "ri"], W[p + "ri.b"])
    log_a = -8.0 * r * softplus(W[p + "lam"])
    a = np.exp(log_a)
    drive = np.sqrt(1.0 - a * a) * i * u
    S = np.zeros(u.shape[1])
    out = np.empty_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + drive[t]
        out[t] = S
    return rounder(out * y) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ attention
def pair_angles(positions, pairs, base, dims):
    f = base ** (-2.0 * np.arange(pairs) / dims)
    return np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]


def rotate_halves(v, positions, dims, base, sign=1.0):
    """Turn pairs (i, i + dims/2) of the first ``dims`` channels of v [T, heads, channels] by position * base^(-2i/dims)."""
    out = v.copy()
    half = dims // 2
    ang = sign * pair_angles(positions, half, base, dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def visible_blocks(i, size, pool):
    """How many pooled blocks position i sees: block b is seen when its last position b pool + pool - 1 <= i - size."""
    return max(0, (i - size + 1) // pool)


def attend_window_and_blocks(q, k, v, size, pool, scale, cap, temp=None, sink=None, rounder=_same):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] as the cache holds them (positions 0..T-1).  Row i attends over the
    positions j with 0 <= i - j < size and over the means of the blocks of ``pool`` positions that lie wholly before them
    (``pool`` None: none); score = q . k * scale * temp[h], capped by cap * tanh(. / cap) (``cap`` None: not); the
    denominator has the extra term exp(sink[h]) (``sink`` None: not).  Returns [T, H, dv]."""
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    if pool is not None:
        nb = T // pool
        pk = rounder(k[:nb * pool].reshape(nb, pool, G, dk).mean(1))
        pv = rounder(v[:nb * pool].reshape(nb, pool, G, dv).mean(1))
    out = np.zeros((T, H, dv))
    for i in range(T):
        n = visible_blocks(i, size, pool) if pool is not None else 0
        lo = max(0, i - size + 1) if size is not None else 0
        for hh in range(H):
            g = hh // (H // G)
            keys, vals = k[lo:i + 1, g], v[lo:i + 1, g]
            if n:
                keys, vals = np.concatenate([pk[:n, g], keys], axis=0), np.concatenate([pv[:n, g], vals], axis=0)
            s = (keys @ q[i, hh]) * scale * (temp[hh] if temp is not None else 1.0)
            if cap is not None:
                s = cap * np.tanh(s / cap)
            top = s.max() if sink is None else max(s.max(), sink[hh])
            e = np.exp(s - top)
            out[i, hh] = (e @ vals) / (e.sum() + (math.exp(sink[hh] - top) if sink is not None else 0.0))
    return out


def pooled_window_attention(h, positions, W, p, m, rounder=_same):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    assert list(positions) == list(range(T)), "the plain attention keeps no cache: positions count from 0"
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, dk)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, dk)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    q = rounder(rotate_halves(q, positions, rot["dims"], rot["base"]))
    k = rounder(rotate_halves(k, positions, rot["dims"], rot["base"]))
    v = rounder(rotate_halves(v, positions, dv, rot["base"]))       # a value is cached turned by its own position ...
    out = attend_window_and_blocks(q, k, v, m["mask"]["size"], m["mask"]["pool"], m["scale"], m["softcap"], W[p + "temp"],
                                   W[p + "sink"], rounder)
    out = rotate_halves(out, positions, dv, rot["base"], sign=-1.0)  # ... and the sum is turned back by the query's
    gate = sigmoid(h @ W[p + "g"].T)
    return rounder(out.reshape(T, H * dv) * gate) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forward
def clamped_expert(h, gate, up, down, limit, rounder=_same):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return rounder(g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, W, p, mlp):
    """(chosen experts [T, top], weights [T, top]): the largest logits, softmax over the chosen ones only."""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    top = mlp["router"]["top"]
    order = np.argsort(-z, axis=1, kind="stable")[:, :top]
    chosen = np.take_along_axis(z, order, axis=1)
    e = np.exp(chosen - chosen.max(1, keepdims=True))
    return order, e / e.sum(1, keepdims=True)


def expert_mixture(h, W, p, mlp, rounder=_same):
    ids, weights = route(h, W, p, mlp)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    limit = mlp["expert"]["limit"]
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], weights[t]):
            q = f"{p}e{int(e)}."
            out[t] += w * clamped_expert(h[t:t + 1], W[q + "gate"], W[q + "up"], W[q + "down"], limit, rounder)[0]
    if mlp.get("shared") is not None:
        s = clamped_expert(h, W[p + "shared.gate"], W[p + "shared.up"], W[p + "shared.down"], mlp["shared"]["limit"], rounder)
        out += s * sigmoid(h @ W[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------------ model
def layer_runs(cfg):
    """The layers in the order they run, with a flag on the first of every pass through the repeated span."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def layer(x, positions, W, cfg, index, rounder=_same):
    L, eps, p = cfg["layers"][index], cfg["norm"]["eps"], f"l{index}."
    h = rounder(rms(x, eps) * W[p + "norm1"])
    if L["type"] == "rglru":
        x = x + gated_linear_recurrence(h, W, p + "mix.", L["mixer"], rounder)
    elif L["type"] == "attention":
        x = x + pooled_window_attention(h, positions, W, p + "mix.", L["mixer"], rounder)
    else:
        raise ValueError(L["type"])
    if L.get("mlp") is not None:
        h = rounder(rms(x, eps) * W[p + "norm2"])
        x = x + expert_mixture(h, W, p + "mlp.", L["mlp"], rounder)
    return x


def forward(tokens, W, cfg, layer_outputs=None, rounded=False):
    """Logits [T, vocab] of a whole sequence.  ``rounded``: everything a part hands to the next is rounded to bfloat16
    (the yardstick of what 8-bit mantissas between the parts cost by themselves)."""
    rounder = round_bf16 if rounded else _same
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    positions = list(range(len(tokens)))
    x = W["embed"][list(tokens)] * cfg["embedding"]["scale"]
    x0 = x.copy()
    for index, first in layer_runs(cfg):
        if first:
            x = rounder(np.concatenate([x, x0], axis=1)) @ W["loop.in"].T
        x = layer(x, positions, W, cfg, index, rounder)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    h = rounder(rms(x, cfg["norm"]["eps"]) * W["final.norm"])
    return (h @ W["embed"].T) * cfg["logit_scale"]
