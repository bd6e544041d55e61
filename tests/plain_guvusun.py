"""A plain, slow implementation of the Guvusun decoder in float64 numpy: one function per mechanism, written from
the design's equations and sharing nothing with the engine.  It runs a whole sequence at once (no cache, no
batching); the engine's tests compare every way of cutting and batching against it.

The design in this file's notation.  T tokens, width D.

* embedding: x_t = E[tok_t] + B[(tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets] (row `buckets` for t = 0),
  then rms(x) * w_embed_norm;
* layer: x <- rms(alpha x + mixer(x)) w1; x <- rms(alpha x + ff(x)) w2; then the token side input
  x <- x + rms(P (gelu_tanh(G x) * S[tok, slice of the layer])) * w_side;
* mixer: latent attention (see ``latent_attention``); feed-forward: routed experts (see ``routed_experts``);
* output: rms(x) w_final, logits = Head x.

rms(z) = z / sqrt(mean(z^2) + eps).
"""
from __future__ import annotations

import math

import numpy as np


def rms(z, eps):
    return z / np.sqrt((z * z).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def round_bf16(a):
    """Round float64 values to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


# ------------------------------------------------------------------------------------------ embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    tokens = [int(t) for t in tokens]
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets for i in range(len(tokens))]


def embedding(tokens, W, cfg):
    x = W["embed"][list(tokens)]
    bg = cfg.get("embedding", {}).get("bigram")
    if bg is not None:
        x = x + W["bigram"][bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return rms(x, cfg["norm"]["eps"]) * W["embed.norm"]


# ------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    dims, base = rot["dims"], float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc is not None:
        where = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return f, amp


def rotate(v, positions, rot):
    """v [T, ..., n]: the first rot.dims channels of the last axis turn by position (pairs i, i + dims/2)."""
    if rot is None or v.shape[-1] == 0:            # a mixer without a rotated part
        return v
    dims = rot["dims"]
    half = dims // 2
    f, amp = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    c, s = (np.cos(ang) * amp).reshape(shape), (np.sin(ang) * amp).reshape(shape)
    out = v.copy()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ------------------------------------------------------------------------------------------ mixer
def latent_keys(h, positions, W, p, m, eps):
    """What a layer with key/value projections of its own caches: the normalised latent c [T, kv_rank] and the
    rotated key part shared by the heads [T, rot_dim]."""
    r = m["kv_rank"]
    d = h @ W[p + "dkv"].T
    c = rms(d[:, :r], eps) * W[p + "dkv.norm"]
    return c, rotate(d[:, r:], positions, m["rot"])


def latent_attention(h, positions, W, p, m, eps, shared=None, rounder=None):
    """h [T, D] -> (output [T, D], (c, k_rot)).  ``shared``: the (c, k_rot) of the layer named by kv_from.
    ``rounder``: applied where an engine that computes in 16 bits hands values from kernel to kernel."""
    rd = rounder or (lambda z: z)
    T = h.shape[0]
    H, dim, rdim, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rdim)
    q_plain, q_rot = rd(q[..., :dim]), rd(rotate(q[..., dim:], positions, m["rot"]))
    c, k_rot = shared if shared is not None else latent_keys(h, positions, W, p, m, eps)
    c, k_rot = rd(c), rd(k_rot)
    k_plain = rd((c @ W[p + "uk"].T).reshape(T, H, dim))
    v = rd((c @ W[p + "uv"].T).reshape(T, H, vd))
    gate = sigmoid(h @ W[p + "g"].T)                                 # [T, H]
    pos = np.asarray(positions)
    visible = pos[None, :] <= pos[:, None]
    out = np.zeros((T, H, vd))
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        sink = float(W[p + "sink"][hd])
        top = np.maximum(s.max(-1, keepdims=True), sink)
        e = np.exp(s - top)
        w = e / (e.sum(-1, keepdims=True) + np.exp(sink - top))
        out[:, hd] = (w @ v[:, hd]) * gate[:, hd:hd + 1]
    return rd(out.reshape(T, H * vd)) @ W[p + "o"].T, (c, k_rot)


# ------------------------------------------------------------------------------------------ feed-forward
def route(h, W, p, router):
    """Per token the chosen experts (indices among experts + identity outputs) and their weights."""
    n, top = router["experts"] + router.get("identity", 0), router["top"]
    z = h @ W[p + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    choice = s + W[p + "correction"]
    groups = router.get("groups")
    if groups is not None and groups["count"] > 1:
        per = n // groups["count"]
        best = choice.reshape(-1, groups["count"], per).max(-1)
        keep = np.argsort(-best, axis=-1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros_like(best, dtype=bool)
        np.put_along_axis(allowed, keep, True, axis=-1)
        choice = np.where(np.repeat(allowed, per, axis=-1), choice, -np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, chosen, axis=-1)
    w = w / (w.sum(-1, keepdims=True) + 1e-20) * router["scale"]
    return chosen, w


def expert(h, W, p, rounder=None):
    rd = rounder or (lambda z: z)
    return rd(silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_experts(h, W, p, mlp, rounder=None):
    router = mlp["router"]
    chosen, w = route(h, W, p, router)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t], w[t]):
            if e >= router["experts"]:                   # an identity expert
                out[t] += weight * h[t]
            else:
                out[t] += weight * expert(h[t:t + 1], W, f"{p}e{e}.", rounder)[0]
    return out


# ------------------------------------------------------------------------------------------ side input, layer, model
def token_side(x, tokens, W, p, index, dim, eps, rounder=None):
    rd = rounder or (lambda z: z)
    e = W["side.embed"][list(tokens), index * dim:(index + 1) * dim]
    g = rd(gelu_tanh(rd(x) @ W[p + "gate"].T) * e)
    y = g @ W[p + "proj"].T
    return x + rms(y, eps) * W[p + "norm"]


def forward(tokens, W, cfg, positions=None, rounder=None, layer_outputs=None, rounded=False):
    """Logits [T, vocab] of a whole sequence; ``layer_outputs`` (a list) receives the stream after every layer.
    ``rounded``: the twin that rounds to bfloat16 what an engine computing in 16 bits hands from kernel to kernel."""
    if rounded:
        rounder = round_bf16
    rd = rounder or (lambda z: z)
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    positions = list(range(len(tokens))) if positions is None else positions
    x = embedding(tokens, W, cfg)
    kept = {}
    side = cfg.get("token_side")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        src = m.get("kv_from")
        y, kept[i] = latent_attention(rd(x), positions, W, p + "mix.", m, eps, kept[src] if src is not None else None, rounder)
        x = rms(alpha * x + y, eps) * W[p + "norm1"]
        if L.get("mlp") is not None:
            x = rms(alpha * x + routed_experts(rd(x), W, p + "mlp.", L["mlp"], rounder), eps) * W[p + "norm2"]
        if side is not None:
            x = token_side(x, tokens, W, p + "side.", i, side["dim"], eps, rounder)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return rd(rms(x, eps) * W["final.norm"]) @ W["head"].T
