"""Mixers that carry a matrix of state per head from token to token instead of keys and values.

`DecayAttention` ("lightning"): linear attention with a fixed decay per head,
    S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t,
q, k, v = act(W h); the concatenated heads get one RMS norm, a sigmoid gate from h, and W_o.

`Wkv` ("wkv"): RWKV-style time mixing.  Five mixes of h with the previous token's h feed r, k, v, the gate and a
two-matrix bottleneck whose output d gives the decay w = exp(-exp(d + w0)) per token and key channel;
    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,  S_t = diag(w_t) S_{t-1} + k_t v_t^T;
each head's o is divided by its root mean square, then weight, silu gate, W_o.

`Gla` ("gla"): gated linear attention, S_t = diag(w_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, with a decay per token and
key channel w = sigmoid(W_a2 W_a1 h + b)^(1 / tau); each head's o gets an RMS norm with a weight shared by the heads,
then a silu gate and W_o.

`GatedDelta` ("gated_delta"): the delta rule with a decay per token, head and key channel and a step size per token
and head, behind short causal convolutions on q, k and v.  `PairMixer` ("pair"): two mixers side by side.

All keep S in 32-bit per sequence (`StateNeed`), zero when a slot is taken, read at the start of a step and
written at its end by one kernel that walks a sequence's tokens in order (csrc/recurrent.cu); single tokens and
short prompts take that path, a long prompt is cut into chunks that run side by side and are joined by a prefix
over the chunks' states.  The projections are matrix products in the engine's type; decays, the recurrence,
its output and the norms are 32-bit.
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import Mixer, part_class, register
from .linear import linear


CHUNK_TOKENS = 64            # a long prompt is cut into chunks of this many tokens that run side by side
CHUNKED_FROM = 256           # the longest sequence of a step from which that pays


def scan_chunks(batch, device):
    """The step's sequences cut into chunks for `ops.state_scan`, or None where the walk in order serves: single
    tokens, short prompts, and captured steps (whose host lists are not the step's)."""
    cached = getattr(batch, "_scan_chunks", False)
    if cached is not False:
        return cached
    out = None
    n_new = batch.new_tokens
    if n_new and len(n_new) == batch.n_seq and sum(n_new) == batch.n_tokens and max(n_new) >= CHUNKED_FROM:
        import numpy as np
        starts, owners, row = [0], [0], 0
        for n in n_new:
            starts += [row + min(n, a + CHUNK_TOKENS) for a in range(0, n, CHUNK_TOKENS)]
            row += n
            owners.append(len(starts) - 1)
        n_chunks = len(starts) - 1
        host = torch.from_numpy(np.concatenate([starts, np.arange(n_chunks), owners]).astype(np.int32))
        dev = host.pin_memory().to(device, non_blocking=True) if device.type == "cuda" else host
        out = (dev[:n_chunks + 1], dev[n_chunks + 1:2 * n_chunks + 1], dev[2 * n_chunks + 1:], n_chunks)
    batch._scan_chunks = out
    return out


class DecayAttention(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hk, hv = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        d = {"q": TensorDecl((hk, spec.width)), "k": TensorDecl((hk, spec.width)), "v": TensorDecl((hv, spec.width)),
             "g": TensorDecl((hv, spec.width)), "o": TensorDecl((spec.width, hv))}
        if getattr(spec, "norm_weight", True):
            d["norm"] = TensorDecl((hv,), "norm_weight")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if len(spec.decay) != spec.n_heads:
            raise QStreamError(QsError.INVALID_MODEL, f"{len(spec.decay)} decays for {spec.n_heads} heads")
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()    # one product for all four
        self.w_out, self.norm = tensors["o"], tensors.get("norm")
        self.decay = torch.tensor(spec.decay, dtype=torch.float32).to(runtime.device)
        self.position = None
        if getattr(spec, "position", None) is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, runtime)

    def state_need(self):
        s = self.spec
        return StateNeed((s.n_heads, s.value_dim, s.key_dim), torch.float32)

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        hk, hv = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        # a rotation enters the recurrence: q and k then leave their product in 32-bit and are rotated in 32-bit
        p = linear(h, self.w_in, out_dtype=torch.float32 if self.position is not None else None)
        q, k = p[:, :hk], p[:, hk:2 * hk]
        if self.position is not None:
            self.position.apply(q, k, step, s.n_heads, s.n_heads, s.key_dim)
        # the factor on k rides on q: the sums are bilinear in the two
        o = ops.state_scan("decay", q, k, p[:, 2 * hk:2 * hk + hv], step.state(cache_id),
                           b.seq_start, b.seq_slot, b.n_seq, s.n_heads, s.key_dim, s.value_dim,
                           head_decay=self.decay, in_activation=s.activation, chunks=scan_chunks(b, h.device),
                           q_scale=float(getattr(s, "key_scale", 1.0)))
        group = s.value_dim if getattr(s, "norm_per_head", False) else hv
        y = ops.gated_group_norm(o, group, self.norm, p[:, 2 * hk + hv:], getattr(s, "gate_activation", "sigmoid"), s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


MIXES = ("r", "k", "v", "g", "w")


class Wkv(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        n, D, R = spec.n_heads * spec.head_dim, spec.width, spec.decay_rank
        d = {name: TensorDecl((n, D)) for name in ("r", "k", "v", "g")}
        d.update({"o": TensorDecl((D, n)), "w1": TensorDecl((R, D)), "w2": TensorDecl((n, R)),
                  "w0": TensorDecl((n,), "bias"), "u": TensorDecl((spec.n_heads, spec.head_dim), "bias"),
                  "norm": TensorDecl((n,), "norm_weight")})
        d.update({"mu_" + m: TensorDecl((D,), "fraction") for m in MIXES})
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.w = {name: tensors[name] for name in ("r", "k", "v", "g", "o", "w1", "w2")}
        self.w0 = tensors["w0"].float().contiguous()
        self.u, self.norm = tensors["u"].contiguous(), tensors["norm"]
        self.mu = torch.stack([tensors["mu_" + m].float() for m in MIXES]).contiguous()        # [5, D] float32

    def state_need(self):
        s = self.spec
        return {"matrix": StateNeed((s.n_heads, s.head_dim, s.head_dim), torch.float32),
                "last_input": StateNeed((s.width,), self.runtime.dtype)}

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        n = s.n_heads * s.head_dim
        last = step.state(cache_id, "last_input")
        mixed = ops.token_shift(h, self.mu, last, b.tok_slot, b.tok_pos)
        ops.keep_last_rows(last, h, b.seq_start, b.seq_slot, b.n_seq)      # after the shift has read it
        r, k, v = (linear(mixed[i], self.w[name]) for i, name in enumerate(("r", "k", "v")))
        gate = linear(mixed[3], self.w["g"])
        d = linear(linear(mixed[4], self.w["w1"], activation="tanh"), self.w["w2"], self.w0, out_dtype=torch.float32)
        o = ops.state_scan("wkv", r, k, v, step.state(cache_id, "matrix"), b.seq_start, b.seq_slot, b.n_seq,
                           s.n_heads, s.head_dim, s.head_dim, decay_logits=d, bonus=self.u, chunks=scan_chunks(b, h.device))
        y = ops.gated_group_norm(o, s.head_dim, self.norm, gate, "silu", s.eps, h.dtype)
        return linear(y, self.w["o"], None, residuals=residuals, out_dtype=out_dtype)


class Mlstm(Mixer):
    """Matrix memory with exponential gates.  q, k, v and the output gate are one product in the engine's type; the
    two gate projections are a product of their own with a 32-bit result.  `ops.mlstm_gates` turns the log gates into
    the recurrence's factors a_t, b_t with the running maximum m per sequence and head; the scan (the kernel of the
    other matrix-state mixers, in its "gated" form) carries S and, as one more column, the normaliser n; the last
    kernel divides, takes each head's unit RMS, the weight and the sigmoid gate."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hk, hv, H = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim, spec.n_heads
        return {"q": TensorDecl((hk, spec.width)), "k": TensorDecl((hk, spec.width)), "v": TensorDecl((hv, spec.width)),
                "g": TensorDecl((hv, spec.width)), "o": TensorDecl((spec.width, hv)), "norm": TensorDecl((hv,), "norm_weight"),
                "i": TensorDecl((H, spec.width)), "f": TensorDecl((H, spec.width)),
                "i_bias": TensorDecl((H,), "bias"), "f_bias": TensorDecl((H,), "bias")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).contiguous()
        self.b_gates = torch.cat([tensors["i_bias"].float(), tensors["f_bias"].float()]).contiguous()
        self.w_out, self.norm = tensors["o"], tensors["norm"]

    def state_need(self):
        s = self.spec
        return {"matrix": StateNeed((s.n_heads, s.value_dim + 1, s.key_dim), torch.float32),
                "maximum": StateNeed((s.n_heads,), torch.float32)}

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        hk, hv = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        p = linear(h, self.w_in)
        raw = linear(h, self.w_gates, self.b_gates, out_dtype=torch.float32)
        a, w, m = ops.mlstm_gates(raw, s.gate_cap, step.state(cache_id, "maximum"), b.seq_start, b.seq_slot, b.n_seq, s.n_heads)
        o = ops.state_scan("gated", p[:, :hk], p[:, hk:2 * hk], p[:, 2 * hk:2 * hk + hv], step.state(cache_id, "matrix"),
                           b.seq_start, b.seq_slot, b.n_seq, s.n_heads, s.key_dim, s.value_dim + 1, token_decay=a,
                           token_weight=w, q_scale=s.key_dim ** -0.5, chunks=scan_chunks(b, h.device))
        y = ops.mlstm_output(o, m, self.norm, p[:, 2 * hk + hv:], s.n_heads, s.value_dim, s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


class Gla(Mixer):
    """Gated linear attention.  q, k, v, the gate and the first matrix of the decays' bottleneck are one product in the
    engine's type; the bottleneck's second matrix (with its bias) gives the decays' logits in 32-bit; the scan takes
    sigmoid(.)^(1 / tau) of them in 32-bit as it stages a token, decays the state, adds k v^T and reads o (a long prompt:
    its chunks side by side, joined by a prefix over the chunks' states); the last kernel takes each head's RMS norm,
    the weight and the silu gate."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hk, hv, D, R = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim, spec.width, spec.decay_rank
        return {"q": TensorDecl((hk, D)), "k": TensorDecl((hk, D)), "v": TensorDecl((hv, D)), "g": TensorDecl((hv, D)),
                "o": TensorDecl((D, hv)), "norm": TensorDecl((spec.value_dim,), "norm_weight"),
                "a1": TensorDecl((R, D)), "a2": TensorDecl((hk, R)), "a2_bias": TensorDecl((hk,), "bias")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if not spec.tau > 0:
            raise QStreamError(QsError.INVALID_MODEL, f"gla: tau={spec.tau} must be positive")
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.rank = tensors["a1"].shape[0]
        self.w_a2, self.b_a2 = tensors["a2"], tensors["a2_bias"].float().contiguous()
        self.w_out = tensors["o"]
        self.norm = tensors["norm"].repeat(spec.n_heads).contiguous()       # one weight of value_dim, shared by the heads

    def state_need(self):
        s = self.spec
        return StateNeed((s.n_heads, s.value_dim, s.key_dim), torch.float32)

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        hk, hv = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        p = linear(h, self.w_in)
        at = 2 * hk + 2 * hv
        z = linear(p[:, at:at + self.rank], self.w_a2, self.b_a2, out_dtype=torch.float32)
        o = ops.state_scan("gla", p[:, :hk], p[:, hk:2 * hk], p[:, 2 * hk:2 * hk + hv], step.state(cache_id),
                           b.seq_start, b.seq_slot, b.n_seq, s.n_heads, s.key_dim, s.value_dim, decay_logits=z,
                           decay_power=1.0 / float(s.tau), q_scale=s.key_dim ** -0.5, chunks=scan_chunks(b, h.device))
        y = ops.gated_group_norm(o, s.value_dim, self.norm, p[:, 2 * hk + hv:at], "silu", s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


class GatedDelta(Mixer):
    """The gated delta rule: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head.  q, k, v and the
    first matrices of the two bottlenecks are one product in the engine's type; the step sizes' projection and the
    decays' second matrix give 32-bit results.  One kernel runs the short convolutions (with the inputs that earlier
    steps left), silu, the unit norms, the decays and the step sizes, all in 32-bit; the scan walks each sequence in
    order (a long prompt: its chunks side by side, each as a linear map of the state it starts from, joined by a
    prefix over the chunks); the last kernel takes each head's unit RMS, the weight and the sigmoid gate."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        D, H, G, dk, dv, n = spec.width, spec.n_heads, spec.n_qk_heads, spec.key_dim, spec.value_dim, spec.conv_taps
        return {"q": TensorDecl((G * dk, D)), "k": TensorDecl((G * dk, D)), "v": TensorDecl((H * dv, D)),
                "conv_q": TensorDecl((G * dk, n)), "conv_k": TensorDecl((G * dk, n)), "conv_v": TensorDecl((H * dv, n)),
                "b": TensorDecl((H, D)), "A_log": TensorDecl((H,), "bias"), "norm": TensorDecl((dv,), "norm_weight"),
                "a1": TensorDecl((spec.decay_rank, D)), "a2": TensorDecl((H * dk, spec.decay_rank)),
                "dt_bias": TensorDecl((H * dk,), "bias"), "g1": TensorDecl((spec.gate_rank, D)),
                "g2": TensorDecl((H * dv, spec.gate_rank)), "o": TensorDecl((D, H * dv))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_qk_heads:
            raise QStreamError(QsError.INVALID_MODEL, f"{spec.n_heads} heads are no multiple of {spec.n_qk_heads} heads of q and k")
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "a1", "g1")], dim=0).contiguous()
        self.ranks = (tensors["a1"].shape[0], tensors["g1"].shape[0])
        self.w_b, self.w_a2, self.w_g2, self.w_out = tensors["b"], tensors["a2"], tensors["g2"], tensors["o"]
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.a_log = tensors["A_log"].float().contiguous()
        self.conv = tuple(tensors["conv_" + n].contiguous() for n in ("q", "k", "v"))
        self.norm = tensors["norm"].repeat(spec.n_heads).contiguous()       # one weight of value_dim, shared by the heads

    def state_need(self):
        s = self.spec
        need = {"matrix": StateNeed((s.n_heads, s.value_dim, s.key_dim), torch.float32)}
        if s.conv_taps > 1:
            need["conv"] = StateNeed((s.conv_taps - 1, 2 * s.n_qk_heads * s.key_dim + s.n_heads * s.value_dim), self.runtime.dtype)
        return need

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        nq, nv = s.n_qk_heads * s.key_dim, s.n_heads * s.value_dim
        ra, rg = self.ranks
        p = linear(h, self.w_in)
        q, k, v = p[:, :nq], p[:, nq:2 * nq], p[:, 2 * nq:2 * nq + nv]
        at = 2 * nq + nv
        a = linear(p[:, at:at + ra], self.w_a2, self.dt_bias, out_dtype=torch.float32)
        gate = linear(p[:, at + ra:at + ra + rg], self.w_g2, out_dtype=torch.float32)
        beta = linear(h, self.w_b, out_dtype=torch.float32)
        held = step.state(cache_id, "conv") if s.conv_taps > 1 else None
        qo, ko, vo, decay, beta = ops.delta_prepare(q, k, v, *self.conv, held, a, beta, self.a_log, b.tok_slot, b.tok_pos,
                                                    s.n_qk_heads, s.n_heads, s.key_dim, s.value_dim, s.key_dim ** -0.5, s.unit_eps)
        if held is not None:                                # after the convolutions have read it
            ops.conv_state_update(held, q, k, v, nq, nv, s.conv_taps, b.seq_start, b.seq_slot, b.n_seq)
        o = ops.state_scan("delta", qo, ko, vo, step.state(cache_id, "matrix"), b.seq_start, b.seq_slot, b.n_seq,
                           s.n_heads, s.key_dim, s.value_dim, key_decay=decay, token_weight=beta,
                           qk_group=s.n_heads // s.n_qk_heads, chunks=scan_chunks(b, h.device))
        y = ops.gated_group_norm(o, s.value_dim, self.norm, gate, "sigmoid", s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


class PairMixer(Mixer):
    """Two mixers side by side on the same input, each with a cache entry of its own (`cache_id` is a pair):
    left_scale * left(h) + right_scale * right(h).  An arrangement that adds branches with factors of its own asks for
    them with `branches`; `forward` adds them up itself."""

    @classmethod
    def declare(cls, spec):
        d = {}
        for side, sub in (("left.", spec.left), ("right.", spec.right)):
            d.update({side + name: decl for name, decl in part_class("mixer", sub.kind).declare(sub).items()})
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        made = []
        for side, sub in (("left.", spec.left), ("right.", spec.right)):
            mine = {name[len(side):]: t for name, t in tensors.items() if name.startswith(side)}
            made.append(part_class("mixer", sub.kind)(sub, mine, runtime))
        self.left, self.right = made
        self.captures_any_step = all(getattr(p, "captures_any_step", False) for p in made)

    def cached_parts(self):
        return [self.left, self.right]

    def branches(self, h, step, cache_id, out_dtype=None):
        left_id, right_id = cache_id
        return [(float(self.spec.left_scale), self.left.forward(h, step, left_id, out_dtype=out_dtype)),
                (float(self.spec.right_scale), self.right.forward(h, step, right_id, out_dtype=out_dtype))]

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        (c1, y1), (c2, y2) = self.branches(h, step, cache_id, out_dtype=torch.float32)
        out = torch.zeros_like(y1)
        for r in residuals:
            if r is not None:
                ops.rmsnorm(out, None, 0.0, update=r, mult=1.0, want_norm=False)
        ops.rmsnorm(out, None, 0.0, update=y1, mult=c1, want_norm=False)
        ops.rmsnorm(out, None, 0.0, update=y2, mult=c2, want_norm=False)
        return out if out_dtype in (None, torch.float32) or out_dtype == out.dtype else ops.convert(out, out_dtype)


register("mixer", "gated_delta", GatedDelta)
register("mixer", "gla", Gla)
register("mixer", "pair", PairMixer)
register("mixer", "lightning", DecayAttention)
register("mixer", "mlstm", Mlstm)
register("mixer", "wkv", Wkv)
