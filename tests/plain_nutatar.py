"""A plain, slow Nutatar in numpy float64: one function per mechanism, written from the design's equations.

It shares no code with the library: the tests compare the library's kernels, cache and step function with it.
A model is (config dict as in config.json, {tensor name: float64 array}); `forward` runs one whole sequence and
returns the logits of every position (and, if asked, the residual stream after every layer).
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

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def plain_frequencies(dims, base):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])


def yarn_frequencies(dims, base, scaling):
    """The frequencies after YaRN's blend and the factor on cos and sin."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, freq, mag, interleaved):
    """x [T, heads, n]: the first `dims` of the last axis rotated by position * freq; pairs (i, i + dims/2), or
    (2i, 2i + 1) if `interleaved`; cos and sin times `mag`."""
    if not dims:
        return x
    half = dims // 2
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * freq[None, None, :]
    c, s = np.cos(a) * mag, np.sin(a) * mag
    out = x.copy()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def softmax_with_sink(scores, visible, sink_logit):
    """scores [T, T] of one head; `visible` the mask; the denominator holds exp(sink_logit) once more (None: no
    sink).  Returns the weights [T, T]."""
    s = np.where(visible, scores, -np.inf)
    m = s.max(-1, keepdims=True)
    if sink_logit is not None:
        m = np.maximum(m, sink_logit)
    e = np.exp(s - m)
    den = e.sum(-1, keepdims=True)
    if sink_logit is not None:
        den = den + np.exp(sink_logit - m)
    return e / den


# ----------------------------------------------------------------------------- mixers

def attention_mixer(m, w, p, h, eps):
    """Windowed softmax attention with grouped key heads whose values are the keys as projected; one RMS norm over
    the whole q (and k) projection; rotate-half positions on part of each head; a sink of score zero."""
    T = h.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    pos = np.arange(T)
    q = h @ w[p + "q"].T
    k = h @ w[p + "k"].T
    v = k.reshape(T, G, d).copy()
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)
    rot = m.get("rot")
    if rot and rot["dims"]:
        f = plain_frequencies(rot["dims"], rot["base"])
        q = rotate(q, pos, rot["dims"], f, 1.0, False)
        k = rotate(k, pos, rot["dims"], f, 1.0, False)
    size = (m.get("mask") or {}).get("size", 0)
    i, j = pos[:, None], pos[None, :]
    visible = (j <= i) & ((i - j < size) if size else True)
    out = np.zeros((T, H, d))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        out[:, hh] = softmax_with_sink(s, visible, 0.0) @ v[:, g]
    return out.reshape(T, H * d) @ w[p + "o"].T


def latent_of(m, w, p, h, eps):
    """What a latent layer caches: the normed latent c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    r, dr = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms_norm(d[:, :r], w[p + "dkv.norm"], eps)
    rot = m["rot"]
    f, mag = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    kr = rotate(d[:, None, r:r + dr], np.arange(T), rot["dims"], f, mag, True)[:, 0]
    return c, kr


def latent_attention_mixer(m, w, p, h, eps, cached):
    """Causal attention through a latent.  `cached` = (c, k_rot) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = cached
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    rot = m["rot"]
    f, mag = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q_rot = rotate(q[..., dn:], np.arange(T), rot["dims"], f, mag, True)
    k_un = (c @ w[p + "uk"].T).reshape(T, H, dn)
    val = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ w[p + "g"].T)                       # [T, H]
    pos = np.arange(T)
    visible = pos[None, :] <= pos[:, None]
    out = np.zeros((T, H, dv))
    for hh in range(H):
        s = (q[:, hh, :dn] @ k_un[:, hh].T + q_rot[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = (softmax_with_sink(s, visible, float(w[p + "sink"][hh])) @ val[:, hh]) * gate[:, hh:hh + 1]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def gla_mixer(m, w, p, h, eps):
    """Gated linear attention: a decay per token and key channel, the state walked token by token."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, dk)
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward

def dense_ff(w, p, h):
    a = np.maximum(h @ w[p + "up"].T, 0.0)
    return (a * a) @ w[p + "down"].T


def expert(w, p, h, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z, top, count, keep):
    """The chosen experts and their weights for router logits z [T, E]: softmax scores, the best `keep` of `count`
    groups of neighbours by their largest score, then the `top` largest scores inside them."""
    T, E = z.shape
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    per = E // count
    chosen, weights = np.zeros((T, top), dtype=np.int64), np.zeros((T, top))
    for t in range(T):
        group_score = s[t].reshape(count, per).max(-1)
        kept = np.argsort(-group_score, kind="stable")[:keep]
        allowed = np.full(E, -np.inf)
        for g in kept:
            allowed[g * per:(g + 1) * per] = s[t, g * per:(g + 1) * per]
        pick = np.argsort(-allowed, kind="stable")[:top]
        chosen[t], weights[t] = pick, s[t, pick]
    return chosen, weights


def moe_ff(mlp, w, p, h):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h @ w[p + "router"].T, r["top"], groups["count"], groups["keep"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * expert(w, f"{p}e{e}.", h[t:t + 1], mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out += expert(w, p + "shared.", h, mlp["shared"]["limit"])
    return out


# ----------------------------------------------------------------------------- the model

def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one whole sequence; with `want_layers` also the stream after every layer [L, T, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens, dtype=np.int64)] * cfg["embedding"]["scale"]
    cached, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        if kind == "attention":
            y = attention_mixer(m, w, p, x, eps)
        elif kind == "gla":
            y = gla_mixer(m, w, p, x, eps)
        elif kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                cached[i] = latent_of(m, w, p, x, eps)
                src = i
            y = latent_attention_mixer(m, w, p, x, eps, cached[src])
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(w, f"l{i}.mlp.", x) if mlp["kind"] == "dense" else moe_ff(mlp, w, f"l{i}.mlp.", x)
            x = x + rms_norm(y, w[f"l{i}.norm2"], eps)
        after.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(after)) if want_layers else logits


def logits_whole(cfg, w, tokens):
    return forward(cfg, w, tokens)


def greedy(cfg, w, prompt, n_new):
    """The tokens a greedy decoder appends to `prompt`, each step a whole forward pass."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(np.argmax(forward(cfg, w, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
