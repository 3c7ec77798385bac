"""Small Nutatar models for the tests: configurations that differ in every size and option, and weights drawn here
with numpy so that every mechanism carries weight in the logits (decays of the linear attention spread between a half
and nearly one, sinks of the order of the scores, routers far from uniform, clamps that bite)."""
from __future__ import annotations

import json

import numpy as np
import torch

from qstream_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, groups=None, shared=None):
    """groups = (count, keep) or None; shared = (ff, limit) or None."""
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def attention_layer(heads, kv_heads, dim, window, scale, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def gla_layer(heads, dim, vdim, tau, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, scaling=None, kv_from=None, mlp=None):
    """rot = (dims, base); scaling = (factor, original, fast, slow) or None."""
    r = {"dims": rot[0], "base": rot[1]}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": r}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def model(vocab, width, eps, scale, layers):
    return {"architecture": "Nutatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


YARN_A = (8.0, 64, 16.0, 2.0)
# A: every mixer and both feed-forwards, grouped key heads, a window that is no multiple of a page, a rotation over
#    part of the head, two layers that read an earlier layer's latents, a layer without feed-forward, the linear
#    attention first.
CONFIG_A = model(97, 64, 1e-5, 3.0, [
    gla_layer(3, 8, 12, 4.0, mlp=moe(6, 2, 20, 1.0, groups=(3, 2), shared=(24, 2.5))),
    attention_layer(4, 2, 16, 37, 0.3, rot=(8, 1e4), mlp=dense(96)),
    latent_layer(3, 8, 4, 12, 20, 24, 0.35, (4, 500.0), YARN_A, mlp=None),
    latent_layer(2, 12, 4, 8, 16, 24, 0.3, (4, 500.0), YARN_A, kv_from=2, mlp=moe(5, 1, 16, 0.8)),
    attention_layer(2, 2, 8, None, 0.4, rot=(8, 300.0), mlp=dense(40)),
    latent_layer(4, 4, 4, 4, 12, 24, 0.5, (4, 500.0), YARN_A, kv_from=2, mlp=dense(56)),
])
# B: sizes that are no multiples of 8, one head, as many key heads as heads, a window of three and of one, a rotation
#    over the whole head and none at all, frequencies without scaling, every expert chosen, one group, a decay power of one.
CONFIG_B = model(131, 50, 2e-6, 1.0, [
    attention_layer(1, 1, 10, 3, 0.7, rot=(10, 200.0), mlp=moe(4, 4, 14, 2.0, groups=(4, 4), shared=(10, 0.5))),
    gla_layer(5, 6, 4, 1.0, mlp=dense(36)),
    latent_layer(1, 6, 6, 10, 14, 10, 0.6, (6, 1e5), None, mlp=dense(30)),
    attention_layer(3, 3, 6, 1, 0.5, rot=None, mlp=None),
    gla_layer(1, 10, 14, 30.0, mlp=moe(3, 2, 6, 3.0, groups=(1, 1))),
])
# C: sizes that the tensor-core kernels take (multiples of 16), windows of exactly one page and of two, a latent and
#    a rotated part that fill 96 and 128 columns, three experts to a token from two of four groups.
CONFIG_C = model(160, 128, 1e-6, 8.0, [
    latent_layer(4, 32, 32, 32, 64, 64, 0.12, (32, 2e4), (4.0, 128, 8.0, 0.5), mlp=moe(8, 3, 32, 1.2, groups=(4, 2), shared=(48, 1.5))),
    attention_layer(4, 2, 32, 64, 32 ** -0.5, rot=(16, 1e4), mlp=dense(192)),
    gla_layer(2, 64, 32, 16.0, mlp=dense(128)),
    attention_layer(2, 1, 64, 128, 0.125, rot=(64, 5e5), mlp=None),
    latent_layer(2, 64, 32, 64, 48, 64, 0.1, (32, 2e4), (4.0, 128, 8.0, 0.5), kv_from=0, mlp=dense(64)),
    latent_layer(2, 16, 16, 32, 32, 112, 0.2, (16, 1e3), None, mlp=None),
])
# E: wider, for long requests: three query heads to a key head, a window that spans several pages and is no multiple
#    of one, long enough prompts for the scan's chunks, twelve experts.
CONFIG_E = model(400, 320, 1e-6, 12.0, [
    attention_layer(6, 2, 64, 200, 0.1, rot=(32, 1e4), mlp=moe(12, 3, 48, 1.0, groups=(3, 2), shared=(64, 1.5))),
    latent_layer(4, 48, 16, 64, 96, 112, 0.09, (16, 1e5), (16.0, 256, 24.0, 1.5), mlp=dense(320)),
    gla_layer(4, 48, 64, 8.0, mlp=dense(192)),
    latent_layer(8, 32, 16, 32, 64, 112, 0.11, (16, 1e5), (16.0, 256, 24.0, 1.5), kv_from=1, mlp=None),
    attention_layer(3, 3, 80, 70, 0.08, rot=(80, 1e6), mlp=dense(256)),
])
# single mixers: one layer each (the sharing latent layer needs its source), no feed-forward; and the experts alone
CONFIG_T = model(64, 48, 1e-5, 2.0, [attention_layer(4, 2, 8, 23, 0.35, rot=(4, 1e3), mlp=None)])
CONFIG_G = model(64, 48, 1e-5, 2.0, [gla_layer(3, 16, 8, 6.0, mlp=None)])
CONFIG_L = model(64, 48, 1e-5, 2.0, [latent_layer(3, 8, 8, 16, 24, 16, 0.3, (8, 1e3), (2.0, 32, 4.0, 1.0), mlp=None),
                                      latent_layer(2, 16, 8, 8, 12, 16, 0.25, (8, 1e3), (2.0, 32, 4.0, 1.0), kv_from=0, mlp=None)])
CONFIG_M = model(64, 48, 1e-5, 2.0, [gla_layer(1, 4, 4, 2.0, mlp=moe(10, 3, 12, 0.7, groups=(5, 2), shared=(20, 1.0)))])
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "E": CONFIG_E, "T": CONFIG_T, "G": CONFIG_G, "L": CONFIG_L, "M": CONFIG_M}


def make_weights(cfg: dict, seed: int, decay_rank: int = 5, gain_all: float = 1.0) -> dict[str, np.ndarray]:
    """float32 arrays by checkpoint name; the caller rounds them to the stored type.  `gain_all` scales every matrix."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n_out, n_in, gain=1.0):
        return rng.normal(0.0, gain_all * gain / np.sqrt(n_in), size=(n_out, n_in))

    def around_one(n):
        return 1.0 + rng.normal(0, 0.2, n)

    # the embedding's rows are of the order of one after the scale, so that the sublayers (which read the stream as
    # it is) meet inputs of a size that does not depend on the configuration
    w = {"embed": rng.normal(0, 1.0 / cfg["embedding"]["scale"], (V, D)), "final.norm": around_one(D), "head": mat(V, D)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        w[f"l{i}.norm1"] = around_one(D) * 0.7
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            w[p + "q"], w[p + "k"], w[p + "o"] = mat(H * d, D, 2.0), mat(G * d, D, 2.0), mat(D, H * d, 1.5)
            w[p + "q.norm"], w[p + "k.norm"] = around_one(H * d) * 2.0, around_one(G * d) * 2.0
        elif layer["type"] == "gla":
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                w[p + n] = mat(rows, D, 1.5)
            w[p + "o"], w[p + "norm"] = mat(D, H * dv, 1.5), around_one(dv)
            w[p + "a1"], w[p + "a2"] = mat(decay_rank, D, 1.5), mat(H * d, decay_rank, 1.5)
            # sigmoid(z)^(1 / tau) between about a half and nearly one whatever tau: z around log(2^-tau .. ) spread
            tau = m["tau"]
            target = rng.uniform(0.5, 0.9995, H * d)                   # the decay a channel has at z = its bias
            s = np.clip(target ** tau, 1e-9, 1 - 1e-9)
            w[p + "a2.b"] = np.log(s / (1.0 - s))
        else:
            dr, rq, r = m["rot_dim"], m["q_rank"], m["kv_rank"]
            w[p + "dq"], w[p + "dq.norm"], w[p + "uq"] = mat(rq, D, 1.5), around_one(rq), mat(H * (d + dr), rq, 2.0)
            if m.get("kv_from") is None:
                w[p + "dkv"], w[p + "dkv.norm"] = mat(r + dr, D, 1.5), around_one(r)
            w[p + "uk"], w[p + "uv"] = mat(H * d, r, 2.0), mat(H * dv, r, 1.5)
            w[p + "sink"], w[p + "g"], w[p + "o"] = rng.normal(0, 1.5, H), mat(H, D, 2.0), mat(D, H * dv, 1.5)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        w[f"l{i}.norm2"] = around_one(D) * 0.7
        if mlp["kind"] == "dense":
            w[q + "up"], w[q + "down"] = mat(mlp["ff"], D, 1.5), mat(D, mlp["ff"], 1.5)
            continue
        F = mlp["expert"]["ff"]
        w[q + "router"] = mat(mlp["router"]["experts"], D, 3.0)
        for e in range(mlp["router"]["experts"]):
            w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(F, D, 2.0), mat(F, D, 2.0), mat(D, F, 1.5)
        if mlp.get("shared"):
            Fs = mlp["shared"]["ff"]
            w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(Fs, D, 2.0), mat(Fs, D, 2.0), mat(D, Fs, 1.5)
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
    weights = make_weights(cfg, seed + "ABCETGLM".index(which), gain_all=1.0 if dtype == "float32" else 0.5)
    return write_folder(tmp_path / f"nutatar_{which}_{dtype}", cfg, weights, dtype), cfg


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


# float32: rounding of 32-bit sums and exponentials only (typical rows are off by 1e-6); a structural fault moves the
# rows it touches by 3e-2 at least.  bfloat16 (with the gentler weights): a row may be off by a quarter of its spread, a
# request's rows (where there are enough of them for a median to mean something) by 5 % in the median.  A router that
# meets two nearly equal scores may pick the other expert in bfloat16 (random weights bring such a row every hundred
# or so, a top-1 router without a shared expert more, and the rows behind it read what that row left; the plain model
# shows margins of a thousandth there): one row in twenty, and always one, may therefore be off by more.  A fault of a
# bfloat16 kernel moves the median; a fault of the structure fails the float32 runs of the same tests.
F32_LIMIT = 1e-3
BF16_ROW_LIMIT, BF16_MEDIAN_LIMIT, BF16_ROWS_BEYOND = 2.5e-1, 5e-2, 0.05


def assert_close(got, ref, dtype, what=""):
    e = logits_error(got, ref)
    if dtype == "float32":
        assert e.max() <= F32_LIMIT, f"{what}: error {e.max():.3e} of the logits' spread at row {int(e.argmax())} (limit {F32_LIMIT})"
        return
    beyond = int((e > BF16_ROW_LIMIT).sum())
    assert beyond <= max(1, int(BF16_ROWS_BEYOND * len(e))), \
        f"{what}: {beyond} of {len(e)} rows beyond {BF16_ROW_LIMIT} of the logits' spread, the worst {e.max():.3e} at row {int(e.argmax())}"
    if len(e) >= 16:
        assert np.median(e) <= BF16_MEDIAN_LIMIT, f"{what}: median error {np.median(e):.3e} of the logits' spread"
