"""Nutatar's configuration, read from its own config.json keys.

A Nutatar model lists its layers: `layers[i]` names the layer's mixer (`type`: "attention", "gla" or
"latent_attention"), the mixer's sizes and constants (`mixer`), and its feed-forward (`mlp`: {"kind": "dense", "ff": n},
{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "groups": {"count", "keep"}}, "shared":
{"ff", "limit"} or absent}, or null).  Around them: `vocab`, `width`, `norm.eps`, `embedding.scale`.  Every size and
constant comes from these keys; the rank of the bottleneck behind a gla mixer's decays is taken from the checkpoint's
tensors (a model made here writes it as `mixer.decay_rank`).  The residual stream is 32-bit; the sublayers read it as
it is and a norm meets their results only; the head has a matrix of its own.  The model names no longest sequence;
`max_positions` (the library's own key, default 32,768) bounds the tables of rotation angles and the engine's context.

Mixers:
  "attention": softmax attention inside a sliding window (`mask.size`; absent or 0: all keys) with grouped key heads
      whose values are the keys as projected (no W_v), one RMS norm over the whole q and the whole k projection,
      rotate-half positions on the first `rot.dims` dims of each head, `scale` on the scores, and a sink of score zero
      in every softmax's denominator.
  "gla": gated linear attention with a decay per token and key channel, sigmoid(.)^(1 / `tau`).
  "latent_attention": causal attention through a cached latent (`q_rank`, `kv_rank`, `rot_dim`), interleaved rotary
      pairs with YaRN-scaled frequencies (`rot.scaling`), a learned sink and a sigmoid gate per head; `kv_from`: the
      layer reads the latents of an earlier layer with maps of its own.

Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.<name>`, `l<i>.mlp.<name>`, `final.norm`, `head`; linear weights
are [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import QsError
from .lutelorn import _bad, _get, _positive_int
from .specs import (AttentionSpec, BlockSpec, GlaSpec, HeadSpec, LatentAttentionSpec, LayerRun, MlpSpec, ModelSpec,
                    PairEmbeddingSpec, PositionHalfSpec, RotaryHalfSpec, RoutedExpertsSpec, StreamNormSpec)

MIXERS = ("attention", "gla", "latent_attention")
DEFAULT_MAX_POSITIONS = 32768
# fixed by the design
SINK_SCORE = 0.0            # the windowed attention's sink: one more term exp(0) in the denominator
GLU_ALPHA = 1.702           # an expert's gate is g sigmoid(GLU_ALPHA g)
GLU_SHIFT = 1.0             # and multiplies (u + GLU_SHIFT)


def _number(d, key, what, optional=False, default=None):
    v = _get(d, key, what, (int, float), optional, default)
    return None if v is None else float(v)


def _check_rot(m, what, within, scaled):
    rot = _get(m, "rot", what, dict, optional=not scaled, default=None)
    if rot is None:
        return
    dims = _get(rot, "dims", what + ".rot", int)
    if dims < 0 or dims % 2 or dims > within or not _number(rot, "base", what + ".rot") > 0:
        raise _bad(f"{what}.rot: dims={dims} must be even and within {within}, base positive")
    sc = rot.get("scaling")
    if sc is not None:
        if not scaled:
            raise _bad(f"{what}.rot.scaling: this mixer's rotation is not scaled", QsError.UNSUPPORTED_ARCH)
        for key in ("factor", "original", "fast", "slow"):
            if not _number(sc, key, what + ".rot.scaling") > 0:
                raise _bad(f"{what}.rot.scaling.{key} must be positive")


@dataclass(frozen=True)
class NutatarConfig:
    vocab: int
    width: int
    layers: tuple                       # the config's own layer objects (dicts), checked
    eps: float
    embedding_scale: float
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Nutatar"
    model_type = "nutatar"

    # ----------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict) -> "NutatarConfig":
        layers = _get(d, "layers", "config", list)
        if not layers:
            raise _bad("'layers' is empty")
        emb = _get(d, "embedding", "config", dict, optional=True, default={})
        layers = [copy.deepcopy(layer) for layer in layers]
        for layer in layers:                            # a layer that reads another's latents may leave their sizes to that layer
            m = layer.get("mixer") if isinstance(layer, dict) else None
            src = m.get("kv_from") if isinstance(m, dict) else None
            if isinstance(src, int) and not isinstance(src, bool) and 0 <= src < len(layers) and isinstance(layers[src], dict) \
                    and isinstance(layers[src].get("mixer"), dict):
                for key in ("kv_rank", "rot_dim", "rot"):
                    if key not in m and key in layers[src]["mixer"]:
                        m[key] = copy.deepcopy(layers[src]["mixer"][key])
        cfg = cls(vocab=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
                  layers=tuple(layers),
                  eps=_number(_get(d, "norm", "config", dict), "eps", "norm"),
                  embedding_scale=_number(emb, "scale", "embedding", optional=True, default=1.0),
                  max_positions=_positive_int(d, "max_positions", "config", optional=True, default=DEFAULT_MAX_POSITIONS))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise _bad(f"norm.eps={self.eps} must be positive")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            kind = _get(layer, "type", what, str)
            if kind not in MIXERS:
                raise _bad(f"{what}.type '{kind}' is not one of {MIXERS}", QsError.UNSUPPORTED_ARCH)
            m = _get(layer, "mixer", what, dict)
            what += ".mixer"
            heads, dim = _positive_int(m, "heads", what), _positive_int(m, "dim", what)
            vdim = _positive_int(m, "vdim", what, optional=True, default=dim)
            if kind == "attention":
                kv = _positive_int(m, "kv_heads", what, optional=True, default=heads)
                if heads % kv:
                    raise _bad(f"{what}: {heads} heads are no multiple of {kv} kv_heads")
                if vdim != dim:
                    raise _bad(f"{what}: the values are the keys, so vdim={vdim} must equal dim={dim}")
                _number(m, "scale", what)
                _check_rot(m, what, dim, scaled=False)
                mask = _get(m, "mask", what, dict, optional=True, default={})
                if _get(mask, "size", what + ".mask", int, optional=True, default=0) < 0:
                    raise _bad(f"{what}.mask.size must not be negative")
            elif kind == "gla":
                if not _number(m, "tau", what) > 0:
                    raise _bad(f"{what}.tau must be positive")
            else:
                for key in ("q_rank", "kv_rank", "rot_dim"):
                    _positive_int(m, key, what)
                _number(m, "scale", what)
                _check_rot(m, what, m["rot_dim"], scaled=True)
                src = m.get("kv_from")
                if src is not None:
                    ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
                    other = self.layers[src] if ok else None
                    if not ok or other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise _bad(f"{what}.kv_from={src!r} must name an earlier latent-attention layer with a W_dkv of its own")
                    for key in ("kv_rank", "rot_dim", "rot"):
                        if other["mixer"].get(key) != m.get(key):
                            raise _bad(f"{what}.{key} differs from that of layer {src}, whose cache it reads")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            what = f"layers[{i}].mlp"
            mk = _get(mlp, "kind", what, str)
            if mk == "dense":
                _positive_int(mlp, "ff", what)
            elif mk == "moe":
                ex = _get(mlp, "expert", what, dict)
                _positive_int(ex, "ff", what + ".expert")
                _number(ex, "limit", what + ".expert")
                r = _get(mlp, "router", what, dict)
                E, top = _positive_int(r, "experts", what + ".router"), _positive_int(r, "top", what + ".router")
                g = r.get("groups") or {"count": 1, "keep": 1}
                count, keep = _positive_int(g, "count", what + ".router.groups"), _positive_int(g, "keep", what + ".router.groups")
                if E % count or keep > count or keep * (E // count) < top or top > E:
                    raise _bad(f"{what}.router: {E} experts, {count} groups, {keep} kept, top {top} do not fit together")
                if mlp.get("shared") is not None:
                    _positive_int(mlp["shared"], "ff", what + ".shared")
                    _number(mlp["shared"], "limit", what + ".shared")
            else:
                raise _bad(f"{what}.kind '{mk}' is not 'dense' or 'moe'", QsError.UNSUPPORTED_ARCH)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "model_type": self.model_type, "vocab": self.vocab,
                "width": self.width, "layers": [copy.deepcopy(layer) for layer in self.layers],
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                "max_positions": self.max_positions}

    # ----------------------------------------------------------------- the model
    def _norm(self, name: str) -> StreamNormSpec:
        return StreamNormSpec(self.width, self.eps, center=False, names={"weight": name})

    def _mixer_spec(self, i: int, kind: str, m: dict):
        D, p = self.width, f"l{i}.mix."
        heads, dim = m["heads"], m["dim"]
        if kind == "attention":
            rot = m.get("rot")
            position = None
            if rot is not None and rot["dims"] > 0:
                position = PositionHalfSpec(rotary_dim=rot["dims"], base=float(rot["base"]), max_positions=self.max_positions)
            names = {"q": p + "q", "k": p + "k", "q_norm": p + "q.norm", "k_norm": p + "k.norm", "out": p + "o"}
            return AttentionSpec(width=D, n_heads=heads, n_kv_heads=m.get("kv_heads", heads), head_dim=dim, position=position,
                                 window=int((m.get("mask") or {}).get("size", 0)), score_scale=float(m["scale"]),
                                 qk_norm="whole", values_from_keys=True, fixed_sink=SINK_SCORE, eps=self.eps, names=names)
        if kind == "gla":
            names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
            names["a2_bias"] = p + "a2.b"
            return GlaSpec(width=D, n_heads=heads, key_dim=dim, value_dim=m.get("vdim", dim), tau=float(m["tau"]),
                           eps=self.eps, decay_rank=int(m.get("decay_rank", -1)), names=names)
        shares = m.get("kv_from") is not None
        names = {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "uk": p + "uk", "uv": p + "uv", "o": p + "o",
                 "sink": p + "sink", "g": p + "g"}
        if not shares:
            names.update({"dkv": p + "dkv", "dkv_norm": p + "dkv.norm"})
        rot = m["rot"]
        scaling = rot.get("scaling")
        position = RotaryHalfSpec(rotary_dim=rot["dims"], base=float(rot["base"]), layout="interleaved",
                                  scaling={k: float(v) for k, v in scaling.items()} if scaling else None)
        return LatentAttentionSpec(width=D, n_heads=heads, head_dim=dim, rot_dim=m["rot_dim"], v_head_dim=m.get("vdim", dim),
                                   q_rank=m["q_rank"], kv_rank=m["kv_rank"], score_scale=float(m["scale"]), eps=self.eps,
                                   position=position, shares_cache=shares, sink=True, head_gate=True, names=names)

    def _ffn_spec(self, i: int, mlp: dict):
        D, p = self.width, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return MlpSpec(width=D, inner=mlp["ff"], activation="relu2", bias=False, names={"up": p + "up", "down": p + "down"})
        r = mlp["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        names = {"router": p + "router"}
        for e in range(r["experts"]):
            names[f"gate{e}"], names[f"up{e}"], names[f"down{e}"] = f"{p}e{e}.gate", f"{p}e{e}.up", f"{p}e{e}.down"
        shared = mlp.get("shared")
        if shared is not None:
            names.update({"shared_gate_proj": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down"})
        return RoutedExpertsSpec(width=D, n_experts=r["experts"], inner=mlp["expert"]["ff"], top=r["top"], groups=g["count"],
                                 keep=g["keep"], route_scale=1.0, activation=None, scores="softmax", group_score="max",
                                 correction=False, shared_gate=False, gated=True, limit=float(mlp["expert"]["limit"]),
                                 shared_inner=shared["ff"] if shared is not None else 0,
                                 shared_limit=float(shared["limit"]) if shared is not None else 0.0,
                                 glu_alpha=GLU_ALPHA, glu_shift=GLU_SHIFT, names=names)

    def model_spec(self) -> ModelSpec:
        D = self.width
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            norms = {"post_input": self._norm(f"l{i}.norm1")}
            ffn = None
            if layer.get("mlp") is not None:
                norms["post_ffn"] = self._norm(f"l{i}.norm2")
                ffn = self._ffn_spec(i, layer["mlp"])
            blocks.append(BlockSpec(arrangement="post_norm", norms=norms, ffn=ffn,
                                    mixer=self._mixer_spec(i, layer["type"], layer["mixer"])))
            src = layer["mixer"].get("kv_from")
            schedule.append(LayerRun(layer=i, cache=i if src is None else src))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, width=D, max_positions=self.max_positions,
            embedding=PairEmbeddingSpec(vocab_size=self.vocab, width=D, scale=self.embedding_scale, buckets=0,
                                        stream_dtype="float32", names={"weight": "embed"}),
            layers=tuple(blocks), schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=HeadSpec(vocab_size=self.vocab, width=D, bias=False, tied=False, names={"weight": "head"}),
        )
