"""Small Sefuvik models for the tests: configurations that differ in every size and option, and weights drawn here
with numpy so that every mechanism carries weight in the logits (decays of the delta rule spread between a half and
nearly one, sinks and the two maps' weights of the order of the scores, mixing matrices of the stream's copies far
from the identity)."""
from __future__ import annotations

import json

import numpy as np
import torch

from qstream_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def retention_layer(dim, vdim, decay, rot=None, mlp=None):
    m = {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def attention_layer(heads, kv_heads, dim, vdim, window, keep, scale, diff, mlp=None):
    mask = {"size": window}
    if keep is not None:
        mask["keep_first"] = keep
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": mask, "scale": scale, "diff": diff}}


def parallel_layer(left, right, scales=(0.8, 0.9), mlp=None):
    """left = (heads, kv_heads, dim, vdim, chunk, scale, (rot dims, base) or None); right = (heads, kv_heads, dim, vdim, taps)."""
    H, G, d, dv, chunk, scale, rot = left
    lm = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "mask": {"size": chunk}, "scale": scale}
    if rot:
        lm["rot"] = {"dims": rot[0], "base": rot[1]}
    H2, G2, d2, dv2, taps = right
    rm = {"heads": H2, "kv_heads": G2, "dim": d2, "vdim": dv2, "conv": taps}
    return {"type": "parallel", "mlp": mlp, "mixer": {"left": lm, "right": rm, "left_scale": scales[0], "right_scale": scales[1]}}


# A: every mixer, three copies of the stream, grouped heads, values wider and narrower than keys, a rotation over part of
#    the head, a chunk and a window that are no multiples of a page, a layer without feed-forward.
CONFIG_A = {
    "architecture": "Sefuvik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [
        parallel_layer((4, 2, 16, 24, 37, 0.3, (8, 1e4)), (4, 2, 8, 12, 4), (0.7, 1.1), mlp=dense(96)),
        attention_layer(3, 1, 16, 8, 50, 5, 0.25, 0.2, mlp=None),
        retention_layer(8, 16, (0.9, 0.99, 0.999), rot=(4, 500.0), mlp=dense(40)),
        attention_layer(2, 2, 8, 24, 19, 0, 0.4, 0.35, mlp=dense(56)),
        parallel_layer((2, 1, 8, 8, 64, 0.5, None), (2, 2, 16, 8, 2), (1.0, 1.0), mlp=None),
    ],
}
# B: sizes that are no multiples of 8, one copy of the stream (mixing tensors of one element), one head, as many key
#    heads as heads, one tap (no convolution state), a window that keeps more first tokens than it is long, a chunk of
#    three, a retention without rotation and with a rotation over the whole head, no decay at all.
CONFIG_B = {
    "architecture": "Sefuvik", "vocab": 131, "width": 50, "norm": {"eps": 2e-6}, "streams": 1,
    "layers": [
        retention_layer(12, 20, (1.0,), rot=None, mlp=dense(36)),
        parallel_layer((1, 1, 10, 14, 3, 0.7, (10, 200.0)), (5, 5, 6, 4, 1), (0.5, 1.3), mlp=dense(30)),
        attention_layer(1, 1, 10, 6, 7, 11, 0.5, 0.1, mlp=None),
        retention_layer(6, 6, (0.5, 0.97), rot=(6, 1e5), mlp=None),
        parallel_layer((3, 3, 6, 10, 29, 0.6, (4, 50.0)), (3, 1, 10, 14, 5), (1.2, 0.4), mlp=dense(44)),
    ],
}
# C: sizes that tensor-core kernels take (multiples of 16), four copies, a window and a chunk of exactly one page and
#    of two, kept first tokens beyond a page.
CONFIG_C = {
    "architecture": "Sefuvik", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "streams": 4,
    "layers": [
        attention_layer(4, 2, 32, 64, 64, 70, 32 ** -0.5, 0.25, mlp=dense(192)),
        parallel_layer((4, 2, 64, 32, 128, 0.11, (32, 2e4)), (4, 4, 32, 32, 3), (0.75, 0.85), mlp=dense(128)),
        retention_layer(32, 64, (0.9375, 0.998046875), rot=(16, 3e5), mlp=dense(96)),
        parallel_layer((2, 2, 32, 32, 64, 0.2, (32, 1e4)), (2, 1, 64, 64, 4), (1.0, 0.5), mlp=None),
        attention_layer(2, 1, 64, 32, 128, 0, 0.125, 0.25, mlp=dense(64)),
    ],
}
# E: wider, for long requests: head sizes of 32 to 80 that the tensor-core kernels take, three query heads to a key head,
#    a chunk and a window that are no multiples of a page and span several, kept first tokens, long enough prompts for
#    the scans' chunks.
CONFIG_E = {
    "architecture": "Sefuvik", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "streams": 3,
    "layers": [
        parallel_layer((6, 2, 32, 48, 100, 0.2, (16, 1e4)), (4, 2, 48, 32, 4), (0.6, 0.9), mlp=dense(320)),
        attention_layer(6, 2, 32, 80, 150, 9, 0.15, 0.2, mlp=dense(192)),
        retention_layer(48, 64, (0.98, 0.9995, 0.9), rot=(24, 1e5), mlp=dense(256)),
        attention_layer(3, 3, 64, 64, 70, 0, 0.1, 0.35, mlp=None),
    ],
}
# single mixers: one layer each, no feed-forward, one copy
CONFIG_R = {"architecture": "Sefuvik", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "streams": 2,
            "layers": [retention_layer(16, 8, (0.8, 0.995, 1.0), rot=(8, 1e3), mlp=None)]}
CONFIG_D = {"architecture": "Sefuvik", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "streams": 2,
            "layers": [attention_layer(4, 2, 8, 16, 23, 3, 0.35, 0.3, mlp=None)]}
CONFIG_P = {"architecture": "Sefuvik", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "streams": 2,
            "layers": [parallel_layer((4, 1, 8, 8, 21, 0.35, (8, 1e3)), (4, 2, 8, 16, 3), (0.9, 1.1), mlp=None)]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "R": CONFIG_R, "D": CONFIG_D, "P": CONFIG_P, "E": CONFIG_E}


def make_weights(cfg: dict, seed: int, decay_rank: int = 5, gate_rank: int = 7, gain_all: float = 1.0) -> dict[str, np.ndarray]:
    """float32 arrays by checkpoint name; the caller rounds them to the stored type.  `gain_all` scales every matrix:
    with 1 a layer doubles a rounding error that enters it (measured), which 32-bit runs bear and bfloat16 runs do not."""
    rng = np.random.default_rng(seed)
    D, V, S = cfg["width"], cfg["vocab"], cfg["streams"]

    def mat(n_out, n_in, gain=1.0):
        return rng.normal(0.0, gain_all * gain / np.sqrt(n_in), size=(n_out, n_in))

    def around_zero(n):
        return rng.normal(0, 0.2, n)

    w = {"embed": rng.normal(0, 1.0, (V, D)), "embed.norm": around_zero(D), "final.norm": around_zero(D)}

    def attention(p, m, maps, bias):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "q"], w[p + "k"], w[p + "v"] = mat(H * maps * d, D, 2.0), mat(G * maps * d, D, 2.0), mat(G * dv, D, 1.5)
        w[p + "o"] = mat(D, H * dv, 1.5)
        if bias:
            w[p + "q.b"], w[p + "k.b"], w[p + "v.b"] = rng.normal(0, 0.3, H * maps * d), rng.normal(0, 0.3, G * maps * d), rng.normal(0, 0.3, G * dv)

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for q in (1, 2) if layer.get("mlp") else (1,):
            w[p + f"norm{q}"], w[p + f"ls{q}"] = around_zero(D), 1.0 + rng.normal(0, 0.3, D)
            w[p + f"hc{q}.in"] = 1.0 / S + rng.normal(0, 0.3, S)
            w[p + f"hc{q}.out"] = 1.0 + rng.normal(0, 0.3, S)
            w[p + f"hc{q}.mix"] = np.eye(S) * 0.8 + rng.normal(0, 0.25, (S, S))
        if layer["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                w[p + "mix." + n] = mat(rows, D, 1.5)
            w[p + "mix.o"] = mat(D, H * dv, 1.5)
        elif layer["type"] == "attention":
            attention(p + "mix.", m, 2, True)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + n] = rng.normal(0, 0.6 / np.sqrt(m["dim"]) ** 0.5, m["dim"])
        else:
            lp, lm = p + "mix.left.", m["left"]
            attention(lp, lm, 1, False)
            w[lp + "g"], w[lp + "sink"] = mat(lm["heads"] * lm["vdim"], D, 1.5), rng.normal(0, 1.5, lm["heads"])
            rp, rm = p + "mix.right.", m["right"]
            H, G, d, dv, taps = rm["heads"], rm["kv_heads"], rm["dim"], rm["vdim"], rm["conv"]
            w[rp + "q"], w[rp + "k"], w[rp + "v"] = mat(G * d, D, 2.0), mat(G * d, D, 2.0), mat(H * dv, D, 1.5)
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[rp + n + ".conv"] = rng.normal(0, 0.7, (rows, taps))
            w[rp + "b"] = mat(H, D, 2.0)
            w[rp + "a1"], w[rp + "a2"] = mat(decay_rank, D, 1.5), mat(H * d, decay_rank, 1.5)
            w[rp + "g1"], w[rp + "g2"] = mat(gate_rank, D, 1.5), mat(H * dv, gate_rank, 1.5)
            # exp(A_log) softplus(a + dt_bias) between about 0.001 and 1: decays between 0.4 and 0.999
            w[rp + "A_log"], w[rp + "dt_bias"] = rng.uniform(-4.0, -0.5, H), rng.uniform(-3.0, 1.0, H * d)
            w[rp + "norm"], w[rp + "o"] = 1.0 + rng.normal(0, 0.2, dv), mat(D, H * dv, 1.5)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, D, 1.5), mat(F, D, 1.5), mat(D, F, 1.5)
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}


def write_folder(folder, cfg: dict, weights: dict, dtype: str):
    """config.json + model.safetensors with the weights rounded to `dtype`."""
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    write_safetensors(folder / "model.safetensors", {k: torch.from_numpy(np.array(v, dtype=np.float32)).to(dt) for k, v in weights.items()})
    return folder


def make_folder(tmp_path, which: str, dtype: str, seed: int = 0):
    cfg = CONFIGS[which]
    weights = make_weights(cfg, seed + "ABCRDPE".index(which), gain_all=1.0 if dtype == "float32" else 0.4)
    return write_folder(tmp_path / f"sefuvik_{which}_{dtype}", cfg, weights, dtype), cfg


def load_plain(folder):
    """(config dict, {name: float64 array}) of a folder, as the plain model takes them: the stored values exactly."""
    cfg = json.loads((folder / "config.json").read_text())
    f = SafetensorsFile(folder / "model.safetensors")
    try:
        w = {name: f.read(name).to(torch.float64).numpy().copy() for name in f.names()}
    finally:
        f.close()
    return cfg, w


def logits_error(got, ref):
    """Per row: the root mean square of the difference (means taken off) over that of the reference."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all()
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))


# float32: rounding of 32-bit sums and exponentials only, doubled by every layer of these large weights (typical rows
# are off by 5e-6, single ones by 3e-4); a structural fault moves the rows it touches by 3e-2 at least.  bfloat16 (with
# the gentler weights): a single row may be off by a quarter of its spread, a request's rows (where there are enough of them
# for a median to mean something) by 5 % in the median.
F32_LIMIT = 1e-3
BF16_ROW_LIMIT, BF16_MEDIAN_LIMIT = 2.5e-1, 5e-2


def assert_close(got, ref, dtype, what=""):
    e = logits_error(got, ref)
    limit = F32_LIMIT if dtype == "float32" else BF16_ROW_LIMIT
    assert e.max() <= limit, f"{what}: error {e.max():.3e} of the logits' spread at row {int(e.argmax())} (limit {limit})"
    if dtype == "bfloat16" and len(e) >= 16:
        assert np.median(e) <= BF16_MEDIAN_LIMIT, f"{what}: median error {np.median(e):.3e} of the logits' spread"
