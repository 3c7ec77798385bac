"""Causal softmax attention over the sequence's paged cache.

q/k/v projections (QStream src/engine.c:841-867), position encoding on q and k before
the keys are kept (:871-880), scores q.k / sqrt(dh) over the keys up to the token's own
position, softmax, weighted sum of values (:888-922), heads concatenated, output
projection (:926-934).  Query head j reads key head j // (H / Hkv) (:884,889).  The
three projections are one matrix product over the concatenated weights.

Options a spec may switch on, each with its constants as the spec's fields: values with a head size of
their own; a factor on the scores other than head_dim^-1/2; a tanh cap on the scores; values blended
with those that an earlier layer computed for the same token (what is cached is the blend); a sigmoid gate
from the mixer's input on the concatenated heads (its projection rides in the same product as q, k, v); keys seen
only inside the query's chunk of positions, or inside a window that also keeps the sequence's first tokens; a learned
sink per head in the softmax's denominator; two attention maps per head over the same values, joined as a difference
with a unit RMS per head (differential attention); one RMS norm over the whole q and the whole k projection before the
heads are split; values that are the keys as projected (no W_v); a sink of a fixed score without a tensor.
"""
from __future__ import annotations

import torch

from ..cache import KvNeed
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import Mixer, part_class, register
from .linear import linear


class Attention(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        maps = getattr(spec, "maps", 1)
        hq, hkv = spec.n_heads * maps * spec.head_dim, spec.n_kv_heads * maps * spec.head_dim
        ho, hv = spec.n_heads * spec.value_dim, spec.n_kv_heads * spec.value_dim
        d = {"q": TensorDecl((hq, spec.width)), "out": TensorDecl((spec.width, ho))}
        if getattr(spec, "sink", False):
            d["sink"] = TensorDecl((spec.n_heads,), "bias")
        if maps == 2:
            d.update({n: TensorDecl((spec.head_dim,), "bias") for n in ("lq1", "lk1", "lq2", "lk2")})
        if not spec.shares_cache:
            d["k"] = TensorDecl((hkv, spec.width))
            if not getattr(spec, "values_from_keys", False):
                d["v"] = TensorDecl((hv, spec.width))
        if getattr(spec, "qk_norm", None):
            d["q_norm"] = TensorDecl((hq,), "norm_weight")
            if not spec.shares_cache:
                d["k_norm"] = TensorDecl((hkv,), "norm_weight")
        if spec.qkv_bias:
            d["q_bias"] = TensorDecl((hq,), "bias")
            if not spec.shares_cache:
                d["k_bias"] = TensorDecl((hkv,), "bias")
                d["v_bias"] = TensorDecl((hv,), "bias")
        if spec.gate:
            d["gate"] = TensorDecl((ho, spec.width))
        if spec.value_mix is not None:
            d["value_mix"] = TensorDecl((), "fraction")
        if spec.out_bias:
            d["out_bias"] = TensorDecl((spec.width,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_kv_heads:
            raise QStreamError(QsError.INVALID_MODEL,
                               f"{spec.n_heads} query heads are no multiple of {spec.n_kv_heads} key heads")
        if spec.head_dim % 2 or spec.head_dim > 512 or spec.value_dim > 512:
            raise QStreamError(QsError.UNSUPPORTED_ARCH,
                               f"attention kernels take even head sizes up to 512, not {spec.head_dim} / {spec.value_dim}")
        if spec.value_mix not in (None, "first", "blend") or (spec.value_mix and spec.shares_cache):
            raise QStreamError(QsError.INVALID_MODEL, f"attention: value_mix '{spec.value_mix}' does not fit")
        self.values_from_keys = bool(getattr(spec, "values_from_keys", False))
        self.qk_norm = getattr(spec, "qk_norm", None)
        if self.qk_norm not in (None, "whole"):
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"attention: no norm of q and k of kind '{self.qk_norm}'")
        if self.values_from_keys and (spec.value_dim != getattr(spec, "maps", 1) * spec.head_dim or spec.value_mix or spec.qkv_bias):
            raise QStreamError(QsError.INVALID_MODEL, "attention: values taken from the keys have the keys' size, no bias and no blend")
        names = ["q"] if spec.shares_cache else (["q", "k"] if self.values_from_keys else ["q", "k", "v"])
        mats = [tensors[n] for n in names] + ([tensors["gate"]] if spec.gate else [])
        if len({m.dtype for m in mats}) != 1:
            raise QStreamError(QsError.INVALID_MODEL, "q/k/v projections are stored in different types")
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.b_qkv = None
        if spec.qkv_bias:
            biases = [tensors[n + "_bias"].float() for n in names]
            if spec.gate:                               # the gate's rows of the product have no bias
                biases.append(torch.zeros(tensors["gate"].shape[0], dtype=torch.float32, device=biases[0].device))
            self.b_qkv = torch.cat(biases).contiguous()
        # the blend's weight is a constant of the model: read once, passed to the kernel by value
        self.value_mix = float(tensors["value_mix"].float().item()) if spec.value_mix == "blend" else 0.0
        self.w_out = tensors["out"]
        self.b_out = tensors.get("out_bias") if spec.out_bias else None
        self.maps = int(getattr(spec, "maps", 1))
        self.chunk, self.keep_first = int(getattr(spec, "chunk", 0)), int(getattr(spec, "keep_first", 0))
        if self.maps not in (1, 2) or (self.maps == 2 and (spec.gate or spec.value_mix or spec.shares_cache)):
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"attention: {self.maps} maps per head with these options")
        if self.chunk and spec.window:
            raise QStreamError(QsError.INVALID_MODEL, "attention: chunks and a window exclude each other")
        self.sink = tensors["sink"].float().contiguous() if getattr(spec, "sink", False) else None
        if getattr(spec, "fixed_sink", None) is not None:
            if self.sink is not None:
                raise QStreamError(QsError.INVALID_MODEL, "attention: a learned sink and a fixed one exclude each other")
            self.sink = torch.full((spec.n_heads,), float(spec.fixed_sink), dtype=torch.float32, device=runtime.device)
        self.q_norm = tensors["q_norm"] if self.qk_norm else None
        self.k_norm = tensors["k_norm"] if self.qk_norm and not spec.shares_cache else None
        # which of the kernels' options only the generic kernel offers
        self.masked = bool(self.chunk or self.keep_first or self.sink is not None or self.maps > 1)
        self.lam = 0.0
        if self.maps == 2:                              # a constant of the model: read once, passed to the kernel by value
            import math
            dot = lambda a, b: float((tensors[a].double() * tensors[b].double()).sum().item())    # noqa: E731
            self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + float(spec.diff)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, runtime)

    @property
    def cache_bytes_per_key(self) -> int:
        """What one key of a sequence costs a decode step to read: its key and its value, all heads."""
        return self.spec.n_kv_heads * (self.maps * self.spec.head_dim + self.spec.value_dim) * self.w_qkv.element_size()

    def kv_need(self):
        if self.spec.shares_cache:
            return None
        s = self.spec
        key_dim = self.maps * s.head_dim                # a cached key row holds every map's key
        return KvNeed(n_kv_heads=s.n_kv_heads, head_dim=key_dim, window=s.window,
                      v_head_dim=0 if s.value_dim == key_dim else s.value_dim, chunk=self.chunk, keep_first=self.keep_first)

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        o = self.forward_hidden(h, step, cache_id)
        return linear(o, self.w_out, self.b_out, residuals=residuals, out_dtype=out_dtype)

    # A parallel block may fuse this part's output projection with the feed-forward's down projection:
    # it takes the projection from `output_projection()` and calls `forward_hidden` with a view to fill.
    def output_projection(self):
        return self.w_out, self.b_out

    def forward_hidden(self, h, step, cache_id, out=None):
        """Everything before the output projection: [T, n_heads * value_dim], written to `out` if given."""
        s = self.spec
        b = step.batch
        view = step.kv(cache_id)
        hq, hkv, hv = s.n_heads * self.maps * s.head_dim, s.n_kv_heads * self.maps * s.head_dim, s.n_kv_heads * s.value_dim
        qkv = linear(h, self.w_qkv, self.b_qkv)
        q = qkv[:, :hq]
        table = getattr(self.position, "fused_table", None) if self.position is not None else None
        # the norms over the whole q and k, the rotation and the cache write as one kernel (a rotation that offers no
        # table of angles: norms by themselves, then the rotation's own way)
        fused_norm = bool(self.qk_norm) and (self.position is None or table is not None) and self.maps == 1 and not s.value_mix
        if self.qk_norm and not fused_norm:             # one norm over all heads' rows at once, statistics in 32-bit
            q = ops.rmsnorm(q, self.q_norm, float(s.eps), out_dtype=q.dtype)
        if s.gate and out is not None:
            raise QStreamError(QsError.INVALID_INPUT, "attention: a gated mixer writes its own output")
        half = bool(getattr(self.position, "half_layout", False))
        if self.maps > 1 and self.position is not None:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, "attention: several maps per head with a rotation")
        if fused_norm:
            shares = s.shares_cache
            k = None if shares else qkv[:, hq:hq + hkv]
            v = None if shares else (k if self.values_from_keys else qkv[:, hq + hkv:hq + hkv + hv])
            ops.norm_rope_store(q, k, v, self.q_norm, self.k_norm, float(s.eps), s.n_heads, s.n_kv_heads, s.head_dim,
                                getattr(self.position, "rotary_dim", 0), table, b.tok_slot, b.tok_pos, view.page_table,
                                view.page_tokens, None if shares else view.k, None if shares else view.v, step.status,
                                v_head_dim=s.value_dim, half_layout=half)
        elif s.shares_cache:
            if self.position is not None:
                if table is None:
                    self.position.apply(q, None, step, s.n_heads, s.n_kv_heads, s.head_dim)
                else:                                   # rotate q only: no keys of its own
                    ops.rope_store(q, None, None, s.n_heads, 0, s.head_dim, self.position.rotary_dim, table,
                                   b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, None, None,
                                   step.status, settled=True, half_layout=half)
        else:
            k = qkv[:, hq:hq + hkv]
            v = k if self.values_from_keys else qkv[:, hq + hkv:hq + hkv + hv]     # the keys as projected: the kernel only reads k
            if self.qk_norm:
                k = ops.rmsnorm(k, self.k_norm, float(s.eps), out_dtype=k.dtype)
            v_first = None
            if s.value_mix == "first":
                step.scratch["value_mix"] = v               # later layers of this step blend their values with these
            elif s.value_mix == "blend":
                v_first = step.scratch.get("value_mix")
                if v_first is None or v_first.shape != v.shape:
                    raise QStreamError(QsError.INVALID_MODEL, "attention: values to blend with, but no earlier layer kept any of this shape")
            if self.position is not None and table is None:
                self.position.apply(q, k, step, s.n_heads, s.n_kv_heads, s.head_dim)
            ops.rope_store(q, k, v, s.n_heads * self.maps, s.n_kv_heads, self.maps * s.head_dim if self.maps > 1 else s.head_dim,
                           getattr(self.position, "rotary_dim", 0) if table is not None else 0, table,
                           b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, view.k, view.v,
                           step.status, settled=True,     # a step's slots, positions and pages arrive before its first kernel
                           v_head_dim=s.value_dim, v_first=v_first, v_mix=self.value_mix, half_layout=half)
        gate = qkv[:, qkv.shape[1] - s.n_heads * s.value_dim:] if s.gate else None
        if not self.masked:
            return attend(q, s, step, view, out, gate=gate)
        return self._attend_masked(q, step, view, out, gate)

    def _attend_masked(self, q, step, view, out, gate):
        """Chunks, kept first tokens, sinks and pairs of maps: the bfloat16 engine's decode and prefill kernels take
        them as options (the gate in their last stage), every other case goes to the generic kernel; every softmax
        in 32-bit; the two maps' results stay in 32-bit until their difference has been normed."""
        s, b = self.spec, step.batch
        two = self.maps == 2
        wide = torch.float32 if two else None
        o = None
        if q.dtype == torch.bfloat16:
            from ..csrc import attention_bf16
            o = attention_bf16.attend(q, s, step, view, None if two else out, gate, sink=self.sink, out_dtype=wide)
            if o is not None:
                gate = None                                 # applied by the kernel
        if o is None:
            o = ops.attention(q, s.n_heads * self.maps, s.n_kv_heads, s.head_dim, s.scale, s.window, b.tok_slot, b.tok_pos,
                              view.page_table, view.page_tokens, view.k, view.v, step.status, out=None if two or gate is not None else out,
                              v_head_dim=s.value_dim, softcap=s.softcap, chunk=self.chunk, keep_first=self.keep_first,
                              sink=self.sink, maps=self.maps, out_dtype=wide)
        if two:
            o = ops.pair_diff_norm(o, s.n_heads, s.value_dim, self.lam, 1.0 - float(s.diff), float(s.eps), q.dtype)
        if gate is not None:
            o = ops.gated_group_norm(o, 0, None, gate, "sigmoid", 0.0, o.dtype)
        if out is not None and o.data_ptr() != out.data_ptr():
            out.copy_(o)
            return out
        return o


def attend(q, spec, step, view, out=None, gate=None, sink=None):
    """Pick the attention kernel for this step: decode and prefill have their own
    bfloat16 kernels; the generic kernel takes every other case.  `gate` [T, heads * value_dim]: the result
    times sigmoid(gate), in the bfloat16 kernels' last stage or by a kernel of its own.  `sink` (float32, one per
    query head): exp(sink) joins each softmax's denominator."""
    b = step.batch
    if q.dtype == torch.bfloat16:
        from ..csrc import attention_bf16
        done = attention_bf16.attend(q, spec, step, view, out, gate, sink=sink)
        if done is not None:
            return done
    o = ops.attention(q, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.scale, spec.window,
                      b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, view.k, view.v,
                      step.status, out=out, v_head_dim=spec.value_dim, softcap=spec.softcap, sink=sink)
    if gate is not None:
        o = ops.gated_group_norm(o, 0, None, gate, "sigmoid", 0.0, o.dtype)
    return o


register("mixer", "attention", Attention)
