"""Sefuvik's configuration, read from its own config.json keys.

A Sefuvik model lists its layers: `layers[i]` names the layer's mixer (`type`: "retention", "attention" or
"parallel"), the mixer's sizes and constants (`mixer`), and its feed-forward (`mlp`: {"kind": "dense", "ff": n} or
null).  Around them: `vocab`, `width`, `norm.eps` and `streams`, the number of copies the residual stream is kept in
(absent: one copy and the plain residual sum, no `hc*` tensors).  Every size and constant comes from these keys; the
ranks of the two bottlenecks of a gated delta rule are taken from the checkpoint's tensors (a model made here writes
them as `decay_rank` and `gate_rank`).  The embedding is followed by a norm, norm weights are stored around zero, the
residual stream is 32-bit, every sublayer's result is multiplied by a vector of the width (`ls1`, `ls2`), and the head
is the embedding table.  The model names no longest sequence; `max_positions` (the library's own key, default 32,768)
bounds the tables of rotation angles and the engine's context.

Mixers:
  "retention": linear attention with a fixed decay per head (`decay`), rotated q and k (`rot`), a unit RMS per head,
      a silu gate.
  "attention": differential attention (two maps per head over the same values, `diff`), biases on q, k, v, a sliding
      window (`mask.size`) that keeps the first `mask.keep_first` tokens, `scale` on the scores.
  "parallel": `left`, grouped softmax attention inside chunks of `mask.size` positions with a sink per head, rotated
      (`rot`), gated; beside `right`, the gated delta rule with short convolutions (`conv` taps); the results are
      added with `left_scale` and `right_scale`.

Tensor names: `embed`, `embed.norm`, `l<i>.norm1|norm2`, `l<i>.ls1|ls2`, `l<i>.hc1|hc2.in|out|mix`,
`l<i>.mix.<name>` (`l<i>.mix.left|right.<name>`), `l<i>.mlp.gate|up|down`, `final.norm`; linear weights are [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from ..errors import QsError
from .lutelorn import _bad, _get, _positive_int
from .specs import (AttentionSpec, BlockSpec, DecayAttentionSpec, GatedDeltaSpec, GatedMlpSpec, HeadSpec,
                    HyperConnectionSpec, LayerRun, ModelSpec, NormedEmbeddingSpec, PairMixerSpec, PositionHalfSpec,
                    RmsNormSpec, StreamSumNormSpec)

MIXERS = ("retention", "attention", "parallel")
DEFAULT_MAX_POSITIONS = 32768
UNIT_EPS = 1e-6             # inside the root when q and k of the delta rule are made unit vectors: fixed by the design


def _number(d, key, what, optional=False, default=None):
    v = _get(d, key, what, (int, float), optional, default)
    return None if v is None else float(v)


def _check_rot(m, what, dim):
    rot = m.get("rot")
    if rot is None:
        return
    dims = _get(rot, "dims", what + ".rot", int)
    base = _number(rot, "base", what + ".rot")
    if dims < 0 or dims % 2 or dims > dim or not base > 0:
        raise _bad(f"{what}.rot: dims={dims} must be even and within dim={dim}, base={base} positive")


def _check_heads(m, what):
    heads, dim = _positive_int(m, "heads", what), _positive_int(m, "dim", what)
    kv = _positive_int(m, "kv_heads", what, optional=True, default=heads)
    _positive_int(m, "vdim", what, optional=True, default=dim)
    if heads % kv:
        raise _bad(f"{what}: {heads} heads are no multiple of {kv} kv_heads")
    return heads, dim


def _mask(m, what):
    mask = _get(m, "mask", what, dict, optional=True, default={})
    size = _get(mask, "size", what + ".mask", int, optional=True, default=0)
    keep = _get(mask, "keep_first", what + ".mask", int, optional=True, default=0)
    if size < 0 or keep < 0:
        raise _bad(f"{what}.mask: size={size} and keep_first={keep} must not be negative")
    return size, keep


@dataclass(frozen=True)
class SefuvikConfig:
    vocab: int
    width: int
    layers: tuple                       # the config's own layer objects (dicts), checked
    eps: float
    streams: Optional[int]              # None: one copy, no mixing tensors
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Sefuvik"
    model_type = "sefuvik"

    # ----------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict) -> "SefuvikConfig":
        layers = _get(d, "layers", "config", list)
        if not layers:
            raise _bad("'layers' is empty")
        cfg = cls(vocab=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
                  layers=tuple(copy.deepcopy(layer) for layer in layers),
                  eps=_number(_get(d, "norm", "config", dict), "eps", "norm"),
                  streams=_positive_int(d, "streams", "config", optional=True, default=None),
                  max_positions=_positive_int(d, "max_positions", "config", optional=True, default=DEFAULT_MAX_POSITIONS))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise _bad(f"norm.eps={self.eps} must be positive")
        if self.streams is not None and self.streams > 8:
            raise _bad(f"streams={self.streams}: the kernels take up to 8 copies of the stream", QsError.UNSUPPORTED_ARCH)
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            kind = _get(layer, "type", what, str)
            if kind not in MIXERS:
                raise _bad(f"{what}.type '{kind}' is not one of {MIXERS}", QsError.UNSUPPORTED_ARCH)
            m = _get(layer, "mixer", what, dict)
            what += ".mixer"
            if kind == "retention":
                heads, dim = _check_heads(m, what)
                _check_rot(m, what, dim)
                decay = _get(m, "decay", what, list)
                if len(decay) != heads or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise _bad(f"{what}.decay must list one number per head ({heads})")
            elif kind == "attention":
                _check_heads(m, what)
                _number(m, "scale", what)
                _number(m, "diff", what)
                _mask(m, what)
            else:
                left, right = _get(m, "left", what, dict), _get(m, "right", what, dict)
                _, dim = _check_heads(left, what + ".left")
                _check_rot(left, what + ".left", dim)
                _number(left, "scale", what + ".left")
                _mask(left, what + ".left")
                _check_heads(right, what + ".right")
                taps = _positive_int(right, "conv", what + ".right")
                if taps > 8:
                    raise _bad(f"{what}.right.conv={taps}: the kernels take up to 8 taps", QsError.UNSUPPORTED_ARCH)
                _number(m, "left_scale", what)
                _number(m, "right_scale", what)
            mlp = layer.get("mlp")
            if mlp is not None:
                if _get(mlp, "kind", f"layers[{i}].mlp", str) != "dense":
                    raise _bad(f"layers[{i}].mlp.kind '{mlp['kind']}' is not 'dense'", QsError.UNSUPPORTED_ARCH)
                _positive_int(mlp, "ff", f"layers[{i}].mlp")

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "model_type": self.model_type, "vocab": self.vocab, "width": self.width,
             "layers": [copy.deepcopy(layer) for layer in self.layers], "norm": {"eps": self.eps},
             "max_positions": self.max_positions}
        if self.streams is not None:
            d["streams"] = self.streams
        return d

    # ----------------------------------------------------------------- the model
    def _position(self, m):
        rot = m.get("rot")
        if rot is None or rot["dims"] <= 0:
            return None
        return PositionHalfSpec(rotary_dim=rot["dims"], base=float(rot["base"]), max_positions=self.max_positions)

    def _retention(self, p, m):
        heads, dim = m["heads"], m["dim"]
        return DecayAttentionSpec(width=self.width, n_heads=heads, key_dim=dim, value_dim=m.get("vdim", dim),
                                  decay=tuple(float(x) for x in m["decay"]), eps=self.eps, activation=None,
                                  position=self._position(m), key_scale=dim ** -0.5, norm_per_head=True,
                                  norm_weight=False, gate_activation="silu",
                                  names={n: p + n for n in ("q", "k", "v", "g", "o")})

    def _differential(self, p, m):
        heads, dim = m["heads"], m["dim"]
        size, keep = _mask(m, "mixer")
        names = {"q": p + "q", "k": p + "k", "v": p + "v", "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
                 "out": p + "o", "lq1": p + "lq1", "lk1": p + "lk1", "lq2": p + "lq2", "lk2": p + "lk2"}
        return AttentionSpec(width=self.width, n_heads=heads, n_kv_heads=m.get("kv_heads", heads), head_dim=dim,
                             v_head_dim=m.get("vdim", dim), position=None, qkv_bias=True, score_scale=float(m["scale"]),
                             window=size, keep_first=keep if size else 0, maps=2, diff=float(m["diff"]), eps=self.eps,
                             names=names)

    def _chunked(self, p, m):
        heads, dim = m["heads"], m["dim"]
        size, _ = _mask(m, "mixer")
        names = {"q": p + "q", "k": p + "k", "v": p + "v", "gate": p + "g", "out": p + "o", "sink": p + "sink"}
        return AttentionSpec(width=self.width, n_heads=heads, n_kv_heads=m.get("kv_heads", heads), head_dim=dim,
                             v_head_dim=m.get("vdim", dim), position=self._position(m), score_scale=float(m["scale"]),
                             chunk=size, sink=True, gate=True, names=names)

    def _delta(self, p, m):
        heads, dim = m["heads"], m["dim"]
        names = {n: p + n for n in ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")}
        names.update({"conv_" + n: p + n + ".conv" for n in ("q", "k", "v")})
        return GatedDeltaSpec(width=self.width, n_heads=heads, n_qk_heads=m.get("kv_heads", heads), key_dim=dim,
                              value_dim=m.get("vdim", dim), conv_taps=m["conv"], eps=self.eps, unit_eps=UNIT_EPS,
                              decay_rank=int(m.get("decay_rank", -1)), gate_rank=int(m.get("gate_rank", -1)), names=names)

    def _mixer_spec(self, i, kind, m):
        p = f"l{i}.mix."
        if kind == "retention":
            return self._retention(p, m)
        if kind == "attention":
            return self._differential(p, m)
        return PairMixerSpec(left=self._chunked(p + "left.", m["left"]), right=self._delta(p + "right.", m["right"]),
                             left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))

    def _connection(self, i, q):
        names = {"scale": f"l{i}.ls{q}"}
        if self.streams is not None:
            names.update({n: f"l{i}.hc{q}.{n}" for n in ("in", "out", "mix")})
        return HyperConnectionSpec(streams=self.streams or 1, width=self.width, mixing=self.streams is not None,
                                   layer_scale=True, names=names)

    def model_spec(self) -> ModelSpec:
        D, S = self.width, self.streams or 1
        blocks, schedule, entry = [], [], 0
        for i, layer in enumerate(self.layers):
            norms = {"input": RmsNormSpec(D, self.eps, offset=1.0, names={"weight": f"l{i}.norm1"})}
            connections = {"mixer": self._connection(i, 1)}
            ffn = None
            if layer.get("mlp") is not None:
                norms["post_mixer"] = RmsNormSpec(D, self.eps, offset=1.0, names={"weight": f"l{i}.norm2"})
                connections["ffn"] = self._connection(i, 2)
                ffn = GatedMlpSpec(width=D, inner=layer["mlp"]["ff"], activation="gelu_new",
                                   names={n: f"l{i}.mlp.{n}" for n in ("gate", "up", "down")})
            blocks.append(BlockSpec(arrangement="hyper", norms=norms, connections=connections,
                                    mixer=self._mixer_spec(i, layer["type"], layer["mixer"]), ffn=ffn))
            if layer["type"] == "parallel":             # two parts that keep something: an entry each
                schedule.append(LayerRun(layer=i, cache=(entry, entry + 1)))
                entry += 2
            else:
                schedule.append(LayerRun(layer=i, cache=entry))
                entry += 1
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, width=D, max_positions=self.max_positions,
            embedding=NormedEmbeddingSpec(vocab_size=self.vocab, width=D, eps=self.eps, center=False, offset=1.0,
                                          stream_dtype="float32", names={"weight": "embed", "norm": "embed.norm"}),
            layers=tuple(blocks), schedule=tuple(schedule),
            final_norm=StreamSumNormSpec(D, S, self.eps, offset=1.0, names={"weight": "final.norm"}),
            head=HeadSpec(vocab_size=self.vocab, width=D, bias=False, tied=True, names={}),
        )
