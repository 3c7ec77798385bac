"""A plain, slow Sefuvik in numpy float64: one function per mechanism, written from the design's equations.

It shares no code with the library: the tests compare the library's kernels, cache and step function with it.
A model is (config dict as in config.json, {tensor name: float64 array}); `forward` runs one whole sequence
token by token where a mechanism carries state, and returns the logits of every position (and, if asked, the sum
of the residual streams after every layer).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np

from plain_gptj import read_safetensors


def load_model(folder):
    """(config dict, {tensor name: float64 array}) of a model folder (the reader is `plain_gptj`'s, also test code)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    for f in sorted(folder.glob("*.safetensors")):
        w.update(read_safetensors(f))
    return cfg, w


# ----------------------------------------------------------------------------- small pieces

def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose weight is stored around zero: unit RMS times (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rotate_half(x, positions, dims, base):
    """x [T, heads, n]: the first `dims` of the last axis rotated, element i paired with i + dims/2, by the angle
    position * base^(-2i / dims)."""
    if not dims:
        return x
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * f[None, None, :]
    c, s = np.cos(a), np.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- visibility

def visible_window(i, j, size, keep_first):
    """Causal; of the keys behind it a query reaches the nearest `size` (itself among them) and, whatever their
    distance, those at places below `keep_first`.  size 0: all keys behind it."""
    return j <= i and (not size or i - j < size or j < keep_first)


def visible_chunk(i, j, size):
    """Causal, and only inside the query's own block of `size` places (blocks tile the sequence from its first token);
    size 0: all keys behind it."""
    return j <= i and (not size or i // size == j // size)


def masked_softmax_attention(q, k, v, scale, visible, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G).  `visible(i, j)` says which
    keys a query sees.  `sink` [H]: one more term exp(sink_h) in each softmax's denominator, without key or value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j)]
            s = (k[js, g] @ q[i, h]) * scale
            m = max(s.max(), sink[h]) if sink is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e[:, None] * v[js, g]).sum(0) / den
    return out


# ----------------------------------------------------------------------------- mixers

def retention(m, w, p, h, eps):
    """Linear attention with a fixed decay per head, rotated q and k, no softmax and no denominator."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    rot = m.get("rot") or {}
    pos = np.arange(T)
    q = rotate_half(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_half(k, pos, rot.get("dims", 0), rot.get("base", 1.0)) * d ** -0.5
    o = np.zeros((T, H, dv))
    for hh in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = m["decay"][hh] * S + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S.T @ q[t, hh]
    o = rms_unit(o, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def short_conv(x, taps):
    """Causal convolution over time per channel: x [T, C], taps [C, n]; tap n - 1 weighs the token itself, tap n - 1 - j the token j
    places back; what lies before the sequence counts as zero."""
    T, C = x.shape
    n = taps.shape[1]
    pad = np.concatenate([np.zeros((n - 1, C)), x])
    return sum(pad[j:j + T] * taps[None, :, j] for j in range(n))


def gated_delta(m, w, p, h, eps):
    """The gated delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                                    # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, d))    # [T, H, d]
    o = np.zeros((T, H, dv))
    for hh in range(H):
        gg = hh // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, gg])
            S = S + np.outer(k[t, gg], u)
            o[t, hh] = S.T @ q[t, gg]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    o = rms_unit(o, eps) * w[p + "norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ w[p + "o"].T


def chunked_sink_attention(m, w, p, h):
    """Grouped softmax attention inside chunks, with a sink in the denominator and a sigmoid gate on the heads."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    rot = m.get("rot") or {}
    pos = np.arange(T)
    q = rotate_half(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_half(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    size = (m.get("mask") or {}).get("size", 0)
    o = masked_softmax_attention(q, k, v, m["scale"], lambda i, j: visible_chunk(i, j, size), sink=w[p + "sink"])
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(m, w, p, h, eps):
    left = chunked_sink_attention(m["left"], w, p + "left.", h)
    right = gated_delta(m["right"], w, p + "right.", h, eps)
    return left, right


def differential_attention(m, w, p, h, eps):
    """Two attention maps over the same values, o = a1 - lambda a2, unit RMS per head, times (1 - diff); sliding
    window that also reaches the sequence's first places; biases on q, k, v; positions do not enter."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    mask = m.get("mask") or {}
    size, keep = mask.get("size", 0), mask.get("keep_first", 0)
    see = lambda i, j: visible_window(i, j, size, keep)
    a1 = masked_softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], see)
    a2 = masked_softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], see)
    lam = math.exp(w[p + "lq1"] @ w[p + "lk1"]) - math.exp(w[p + "lq2"] @ w[p + "lk2"]) + m["diff"]
    o = rms_unit(a1 - lam * a2, eps) * (1.0 - m["diff"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ----------------------------------------------------------------------------- the model

def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence (and the sum of the streams after every layer, [layers, T, width])."""
    eps = cfg["norm"]["eps"]
    S = int(cfg.get("streams", 1) or 1)
    x0 = norm_around_zero(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    xs = [x0.copy() for _ in range(S)]
    after = []

    def sublayer(i, q, fn):
        nonlocal xs
        pre = f"l{i}."
        hc = pre + f"hc{q}."
        if hc + "in" in w:
            u = sum(w[hc + "in"][s] * xs[s] for s in range(S))
        else:
            u = xs[0]
        ys = fn(norm_around_zero(u, w[pre + f"norm{q}"], eps))
        ls = w.get(pre + f"ls{q}")
        y = sum(c * (yy * ls if ls is not None else yy) for c, yy in ys)
        if hc + "in" in w:
            xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(S)) + w[hc + "out"][t] * y for t in range(S)]
        else:
            xs = [xs[0] + y]

    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "retention":
            sublayer(i, 1, lambda h: [(1.0, retention(m, w, p, h, eps))])
        elif layer["type"] == "attention":
            sublayer(i, 1, lambda h: [(1.0, differential_attention(m, w, p, h, eps))])
        elif layer["type"] == "parallel":
            sublayer(i, 1, lambda h: list(zip((m["left_scale"], m["right_scale"]), parallel_mixer(m, w, p, h, eps))))
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            sublayer(i, 2, lambda h: [(1.0, feed_forward(w, f"l{i}.mlp.", h))])
        after.append(sum(xs))
    z = norm_around_zero(sum(xs), w["final.norm"], eps)
    logits = z @ w["embed"].T
    return (logits, np.stack(after)) if want_layers else logits


def logits_whole(cfg, w, tokens):
    """Logits [T, vocab] at every position of one sequence."""
    return forward(cfg, w, list(tokens))


def generate_greedy(cfg, w, prompt, max_new_tokens):
    tokens = list(prompt)
    for _ in range(max_new_tokens):
        tokens.append(int(np.argmax(logits_whole(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
