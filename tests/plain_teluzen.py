"""A plain, slow implementation of the Teluzen design: numpy, one function a mechanism, whole
sequences at once (no cache, no batch), in the precision of the arrays it is given (tests pass
float64). It shares nothing with the package: the tests compare the engine with it.

A model is (config, tensors): config.json's dict and {name: array}. Notation: T tokens, W the
model's width, H heads, G key/value heads, d the query/key size of a head, e its value size, S the
window's size, P the tokens of a pooled block.
"""
from __future__ import annotations

import math

import numpy as np


# ---------------------------------------------------------------------------------------- small pieces
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def relu2(z):
    r = np.maximum(z, 0.0)
    return r * r


# ---------------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot):
    """(frequency of every pair [dims/2], the factor on cos and sin). Without `scaling` the
    frequencies are base^(-2i/dims) and the factor is 1. With it (factor, original, fast, slow) the
    slow pairs are stretched by `factor`, the fast ones kept, with a linear ramp between the pairs
    that turn `fast` and `slow` times over `original` positions."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turns_to_pair(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_pair(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_pair(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, rot):
    """x [T, n, d]: of the first rot["dims"] components of every vector, component 2i is paired with
    2i+1 and the pair turned by position * frequency_i; cos and sin carry the scaling's factor."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]               # [T, dims/2]
    c, s = (np.cos(a) * m)[:, None, :], (np.sin(a) * m)[:, None, :]
    out = np.array(x, copy=True)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------------------- who sees whom
def seen_tokens(i, size):
    """The positions a query at position i sees as tokens: the last `size`, its own included."""
    return range(max(0, i - size + 1), i + 1)


def seen_blocks(i, size, pool):
    """The pooled blocks a query at position i sees: block b (positions b*pool .. b*pool+pool-1) when
    its last position is at most i - size."""
    return range(max(0, (i - size + 1) // pool)) if i - size + 1 >= pool else range(0)


def pooled(x, pool):
    """x [T, n, c] -> the means of whole blocks of `pool` positions [T // pool, n, c]."""
    nb = x.shape[0] // pool
    return x[: nb * pool].reshape(nb, pool, *x.shape[1:]).mean(axis=1) if nb else np.zeros((0, *x.shape[1:]), dtype=x.dtype)


def window_pool_weights(q, k, scale, temp, size, pool):
    """Softmax weights of one head. q [T, d], k [T, d] -> (over tokens [T, T], over blocks [T, T // pool]);
    tokens and blocks share the softmax. score = q.k * scale * temp."""
    T = q.shape[0]
    kb = pooled(k[:, None, :], pool)[:, 0]
    wt = np.zeros((T, T), dtype=q.dtype)
    wb = np.zeros((T, kb.shape[0]), dtype=q.dtype)
    for i in range(T):
        tok = list(seen_tokens(i, size))
        blk = list(seen_blocks(i, size, pool))
        s = np.concatenate([k[tok] @ q[i], kb[blk] @ q[i] if blk else np.zeros(0, dtype=q.dtype)]) * scale * temp
        p = np.exp(s - s.max())
        p = p / p.sum()
        wt[i, tok] = p[: len(tok)]
        if blk:
            wb[i, blk] = p[len(tok):]
    return wt, wb


def mix_heads(w, talk):
    """w [H, ...] weights of every head -> sum_g talk[h, g] w[g]."""
    return np.tensordot(talk, w, axes=([1], [0]))


# ---------------------------------------------------------------------------------------- the mixer
def attention_values(h, t, prefix):
    """v = W_v h + b_v as [T, G * e] (before any mixing with the first layer's values)."""
    return h @ t[f"{prefix}.v"].T + t[f"{prefix}.v.b"]


def attention_mixer(h, t, prefix, m, eps, v_first=None):
    """Returns (output [T, W], this layer's values before mixing [T, G e]). `v_first`: the values of
    the first value-mixing layer, or None when this layer does not mix (or is that first layer)."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    S, P = int(m["mask"]["size"]), int(m["mask"]["pool"])
    T = h.shape[0]
    pos = np.arange(T)
    q = h @ t[f"{prefix}.q"].T + t[f"{prefix}.q.b"]
    k = h @ t[f"{prefix}.k"].T + t[f"{prefix}.k.b"]
    v_own = attention_values(h, t, prefix)
    v = v_own
    if v_first is not None:
        lam = float(t[f"{prefix}.vmix"])
        v = (1.0 - lam) * v_own + lam * v_first
    q = rms_norm(q, t[f"{prefix}.q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, t[f"{prefix}.k.norm"], eps).reshape(T, G, d)
    v = v.reshape(T, G, e)
    if m.get("rot"):
        q, k = rotate_neighbours(q, pos, m["rot"]), rotate_neighbours(k, pos, m["rot"])
    vb = pooled(v, P)
    wt = np.zeros((H, T, T), dtype=h.dtype)
    wb = np.zeros((H, T, vb.shape[0]), dtype=h.dtype)
    for a in range(H):
        wt[a], wb[a] = window_pool_weights(q[:, a], k[:, a // (H // G)], float(m["scale"]), float(t[f"{prefix}.temp"][a]), S, P)
    wt, wb = mix_heads(wt, t[f"{prefix}.talk"]), mix_heads(wb, t[f"{prefix}.talk"])
    out = np.zeros((T, H, e), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        out[:, a] = wt[a] @ v[:, g] + wb[a] @ vb[:, g]
    return out.reshape(T, H * e) @ t[f"{prefix}.o"].T, v_own


# ---------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, t, prefix):
    return relu2(h @ t[f"{prefix}.up"].T) @ t[f"{prefix}.down"].T


def gated_expert(h, t, prefix):
    return (silu(h @ t[f"{prefix}.gate"].T) * (h @ t[f"{prefix}.up"].T)) @ t[f"{prefix}.down"].T


def route(h, router, top):
    """(experts [T, top], weights [T, top]): the `top` largest logits (the lower number wins a tie),
    weighted by the softmax over the chosen logits alone."""
    z = h @ router.T
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(z, order, axis=-1)
    p = np.exp(chosen - chosen.max(axis=-1, keepdims=True))
    return order, p / p.sum(axis=-1, keepdims=True)


def moe_ff(h, t, prefix, mlp):
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    which, weight = route(h, t[f"{prefix}.router"], top)
    out = np.zeros((h.shape[0], t[f"{prefix}.e0.down"].shape[0]), dtype=h.dtype)
    for e in range(experts):
        rows, slot = np.nonzero(which == e)
        if rows.size:
            out[rows] += weight[rows, slot][:, None] * gated_expert(h[rows], t, f"{prefix}.e{e}")
    if mlp.get("shared"):
        out = out + gated_expert(h, t, f"{prefix}.shared")
    return out


def feed_forward(h, t, prefix, mlp):
    return dense_ff(h, t, prefix) if mlp["kind"] == "dense" else moe_ff(h, t, prefix, mlp)


# ---------------------------------------------------------------------------------------- the model
def forward(config, t, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0. `layers_out`: a list that receives the
    residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    tokens = np.asarray(tokens)
    T = tokens.shape[0]
    x = t["embed"][tokens] + t["pos"][:T]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        mixes = bool(m.get("v_mix"))
        a, v_own = attention_mixer(rms_norm(x, t[f"l{i}.norm1"], eps), t, f"l{i}.mix", m, eps, v_first if mixes else None)
        if mixes and v_first is None:
            v_first = v_own
        x = x + rms_norm(a, t[f"l{i}.norm1b"], eps)
        if layer.get("mlp"):
            f = feed_forward(rms_norm(x, t[f"l{i}.norm2"], eps), t, f"l{i}.mlp", layer["mlp"])
            x = x + rms_norm(f, t[f"l{i}.norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
