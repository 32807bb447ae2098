"""A plain, slow implementation of the Lokedra design: numpy, one function a mechanism, whole
sequences at once (no cache, no batch), in the precision of the arrays it is given (tests pass
float64). It shares nothing with the package: the tests compare the engine with it.

A model is (config, tensors): config.json's dict and {name: array}. Notation: T tokens, W the
model's width, H heads, G key/value heads, d the query/key size of a head, e its value size.
"""
from __future__ import annotations

import math

import numpy as np


# ---------------------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def token_shift(h, mu):
    """h [T, W]: row t becomes h_t + (h_(t-1) - h_t) * mu, with zeros before the first row."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * mu


def short_conv(x, w):
    """x [T, C], w [C, taps]: y[t] = sum_j w[:, j] x[t - taps + 1 + j], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[: T - back] * w[:, j]
    return y


def stretched_frequencies(rot):
    """The turning rates of the pairs: base^(-2i/dims), each divided by `factor` to the degree its
    wavelength is long (a ramp between the pair that turns `fast` times over `original` positions
    and the one that turns `slow` times), and the magnitude that cos and sin are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])
    number = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(number(float(sc["fast"]))), 0)
    hi = min(math.ceil(number(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, n, d]: the first rot["dims"] components of every vector are turned in neighbouring pairs
    (2i, 2i+1) by the angle position * rate_i; the rest pass."""
    dims = int(rot["dims"])
    f, mag = stretched_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    out = np.array(x, copy=True)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def masked_softmax(scores, visible, one_more=False):
    """scores, visible [T, T]: weights over the visible columns of each row; with `one_more`, 1 joins the
    denominator (a column of score 0 that has no value)."""
    out = np.zeros_like(scores)
    for i in range(scores.shape[0]):
        cols = np.nonzero(visible[i])[0]
        row = scores[i, cols]
        top = max(row.max(), 0.0) if one_more else row.max()
        p = np.exp(row - top)
        out[i, cols] = p / (p.sum() + (math.exp(-top) if one_more else 0.0))
    return out


# ---------------------------------------------------------------------------------------- mixers
def general_delta_recurrence(r, k, v, w, a):
    """One head. r, k, w, a [T, d], v [T, e]. With the unit key u = k / sqrt(sum k^2 + 1e-6):
    S <- diag(w) S - (a u) (u^T S) + k v^T (both first terms read the old S); o = S^T r."""
    T, d = k.shape
    S = np.zeros((d, v.shape[1]), dtype=v.dtype)
    out = np.zeros_like(v)
    for t in range(T):
        u = k[t] / np.sqrt((k[t] * k[t]).sum() + 1e-6)
        S = w[t][:, None] * S - np.outer(a[t] * u, u @ S) + np.outer(k[t], v[t])
        out[t] = S.T @ r[t]
    return out


def general_delta_mixer(h, t, p, m, eps):
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    r, k, v = ((h @ t[f"{p}.{n}"].T).reshape(T, H, d) for n in ("r", "k", "v"))
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ t[f"{p}.w1"].T) @ t[f"{p}.w2"].T + t[f"{p}.w0"])).reshape(T, H, d)
    a = sigmoid(h @ t[f"{p}.a"].T + t[f"{p}.a.b"]).reshape(T, H, d)
    o = np.stack([general_delta_recurrence(r[:, i], k[:, i], v[:, i], w[:, i], a[:, i]) for i in range(H)], axis=1)
    o = rms_unit(o, eps).reshape(T, H * d) * t[f"{p}.norm"] * sigmoid(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


def latent_attention_mixer(h, t, p, m, eps):
    H, d, r, e, kv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = np.arange(T)
    cq = rms_unit(h @ t[f"{p}.dq"].T, eps) * t[f"{p}.dq.norm"]
    q = (cq @ t[f"{p}.uq"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, m["rot"])
    down = h @ t[f"{p}.dkv"].T
    c = rms_unit(down[:, :kv], eps) * t[f"{p}.dkv.norm"]
    k_rot = rotate_pairs(down[:, None, kv:], pos, m["rot"])[:, 0]
    k_plain = (c @ t[f"{p}.uk"].T).reshape(T, H, d)
    v = (c @ t[f"{p}.uv"].T).reshape(T, H, e)
    visible = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, e), dtype=h.dtype)
    for i in range(H):
        s = (q_plain[:, i] @ k_plain[:, i].T + q_rot[:, i] @ k_rot.T) * m["scale"]
        out[:, i] = masked_softmax(s, visible) @ v[:, i]
    return out.reshape(T, H * e) @ t[f"{p}.o"].T


def chunked_attention(h, t, p, m):
    """Grouped queries behind short convolutions; the values are the keys; a position sees the earlier
    positions of its own chunk; 1 joins the softmax's denominator."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = short_conv(h @ t[f"{p}.q"].T + t[f"{p}.q.b"], t[f"{p}.q.conv"]).reshape(T, H, d)
    k = short_conv(h @ t[f"{p}.k"].T + t[f"{p}.k.b"], t[f"{p}.k.conv"]).reshape(T, G, d)
    size = int(m["mask"]["size"])
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    visible = (j <= i) & (i // size == j // size)
    out = np.zeros((T, H, d), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        out[:, a] = masked_softmax((q[:, a] @ k[:, g].T) * m["scale"], visible, one_more=True) @ k[:, g]
    return out.reshape(T, H * d) @ t[f"{p}.o"].T + t[f"{p}.o.b"]


def forget_gate_recurrence(q, f, v):
    """One head. q, f [T, d], v [T, e]: S <- diag(f) S + (1 - f) v^T; o = S^T q."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]), dtype=v.dtype)
    out = np.zeros_like(v)
    for t in range(T):
        S = f[t][:, None] * S + np.outer(1.0 - f[t], v[t])
        out[t] = S.T @ q[t]
    return out


def forget_gate_mixer(h, t, p, m, eps):
    H, d, e = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ t[f"{p}.q"].T).reshape(T, H, d)
    v = (h @ t[f"{p}.v"].T).reshape(T, H, e)
    low = t[f"{p}.lower"]
    f = (low + (1.0 - low) * sigmoid(h @ t[f"{p}.f"].T + t[f"{p}.f.b"])).reshape(T, H, d)
    o = np.stack([forget_gate_recurrence(q[:, i], f[:, i], v[:, i]) for i in range(H)], axis=1)
    o = rms_unit(o, eps) * t[f"{p}.norm"]
    return o.reshape(T, H * e) @ t[f"{p}.o"].T


def parallel_mixer(h, t, p, m, eps):
    return m["left_scale"] * chunked_attention(h, t, f"{p}.left", m["left"]) + m["right_scale"] * forget_gate_mixer(
        h, t, f"{p}.right", m["right"], eps)


MIXERS = {"general_delta": general_delta_mixer, "latent_attention": latent_attention_mixer, "parallel": parallel_mixer}


# ---------------------------------------------------------------------------------------- feed-forward
def route(h, t, p, m):
    """(chosen experts [T, top], their weights [T, top]): softmax over all experts; the choice adds the
    correction, the weights do not, and they are not renormalized."""
    z = h @ t[f"{p}.router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    top = int(m["router"]["top"])
    chosen = np.argsort(-(s + t[f"{p}.correction"]), axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def expert(h, t, p, limit):
    g = np.minimum(h @ t[f"{p}.gate"].T, limit)
    u = np.clip(h @ t[f"{p}.up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[f"{p}.down"].T


def experts_ffn(h, t, p, m):
    chosen, weights = route(h, t, p, m)
    out = np.zeros_like(h)
    limit = float(m["expert"]["limit"])
    for e in range(int(m["router"]["experts"])):
        rows, slot = np.nonzero(chosen == e)
        if rows.size:
            out[rows] += weights[rows, slot][:, None] * expert(h[rows], t, f"{p}.e{e}", limit)
    return out


# ---------------------------------------------------------------------------------------- the model
def layer_runs(config):
    """The layers in the order they run: [(layer, adds the embedding's output first?)]. The layers
    start..stop-1 of `loop` run `times` times in a row; every pass but the first opens with the sum."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or int(loop["stop"]) <= int(loop["start"]):
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for n_pass in range(times):
        runs += [(i, i == start and n_pass > 0) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(config, t, tokens, residuals=None):
    """Logits [T, vocab] of a whole sequence; `residuals`, a list, receives the stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x = t["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    x0 = x
    for i, opens in layer_runs(config):
        if opens:
            x = x + x0
        rec, p = config["layers"][i], f"l{i}"
        h = rms_unit(x, eps) * (1.0 + t[f"{p}.norm1"])
        a = MIXERS[rec["type"]](token_shift(h, t[f"{p}.shift"]), t, f"{p}.mix", rec["mixer"], eps) * t[f"{p}.ls1"]
        if rec.get("mlp") is not None:
            a = a + experts_ffn(h, t, f"{p}.mlp", rec["mlp"]) * t[f"{p}.ls2"]
        x = x + a
        if residuals is not None:
            residuals.append(x)
    return (rms_unit(x, eps) * (1.0 + t["final.norm"])) @ t["embed"].T
