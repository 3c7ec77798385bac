"""How a layer's parts are wired: the arrangements.

"parallel": h = norm(x); x + mixer(h) + ffn(h), one norm, both branches read h.  The
reference engine runs the "sequential" form (x += mixer(norm_1 x); x += ffn(norm_2 x),
QStream src/engine.c:936-948,1173-1174); both are here, built from the same parts.
The residual sum is taken in 32-bit inside the last kernel of the branch that ends
the layer.
"""
from __future__ import annotations

import contextlib

from ..errors import QsError, QStreamError
from .base import Part, part_class, register


class Arrangement(Part):
    role = "arrangement"
    norm_names: tuple = ()
    # the arrangements here read nothing of the step but `decode` and, of a decode step, the number of rows
    # and the longest sequence (which a captured decode step is keyed by)
    captures_own_step = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, {}, runtime)
        self.mixer = parts["mixer"]
        self.ffn = parts["ffn"]
        self.norms = parts["norms"]
        position = getattr(self.mixer, "position", None)
        self.captures_any_step = self.captures_own_step and all(
            getattr(p, "captures_any_step", False)
            for p in (self.mixer, *([self.ffn] if self.ffn is not None else []), *self.norms.values(),
                      *([position] if position else [])))
        missing = [n for n in self.norm_names if n not in self.norms]
        if missing:
            raise QStreamError(QsError.INVALID_MODEL,
                               f"arrangement '{spec.arrangement}' needs the norms {self.norm_names}, "
                               f"the layer lacks {missing}")

    def forward(self, x, step, cache_id):
        raise NotImplementedError

    # What a layer is made of is the arrangement's own business.  The three methods below describe the layers
    # of this library (one mixer, one feed-forward, named norms); an arrangement of another make - two mixers,
    # no feed-forward - overrides them and nothing else in the library changes.
    @classmethod
    def part_specs(cls, spec):
        """Yield (role, part spec) for every part of the layer that holds tensors."""
        yield "mixer", spec.mixer
        yield "feed_forward", spec.ffn
        for norm_spec in spec.norms.values():
            yield "norm", norm_spec

    @classmethod
    def build(cls, spec, make, runtime):
        """Build the layer; `make(role, part_spec)` builds one part with its tensors."""
        parts = {"mixer": make("mixer", spec.mixer), "ffn": make("feed_forward", spec.ffn),
                 "norms": {name: make("norm", ns) for name, ns in spec.norms.items()}}
        return cls(spec, parts, runtime)

    def cached_parts(self):
        """The parts that keep something in the cache (keys and values, or state), in the order of the
        cache entries a schedule run names for this layer: `LayerRun.cache` is one id for one such part, a
        tuple of ids for several; `forward` gets it as it stands."""
        return [self.mixer]


# A decode step runs a parallel block's two branches side by side while the keys and values its rows read
# (rows x the longest sequence x the mixer's bytes per key) stay below this share of the feed-forward's
# weights: then the attention kernels are bound by latency, beyond it by memory like the products.
# Up to 8 rows the two streams' products also share the SMs (see `forward`), which moves the limit up.
# Measured on a B200 against the one fused product, tokens a second, GPT-J-6B's sizes: up to 8 rows +1 to +8 %
# up to a share of 0.5 (1 x 2,048 keys ... 8 x 1,024), -10 % at 0.6 (8 x 1,280); 16 rows and more +6 to +7 % up
# to 0.25 (16 x 256), -5 % at 0.5 (16 x 512).  CodeGen-16B's sizes: +5 to +13 % up to 0.33, +1.5 % at 0.67.
# CodeGen-2B's: +11 to +14 % up to 0.4, -1 to -2 % at 0.8.
SIDE_BRANCH_SHARE = 0.5                 # up to SHARED_SM_ROWS rows
SIDE_BRANCH_SHARE_MANY_ROWS = 0.35      # beyond
SHARED_SM_ROWS = 8


class ParallelBlock(Arrangement):
    """x + mixer(h) + ffn(h).  When both parts end in a projection to the width (they offer
    `output_projection()` and `forward_hidden(..., out=view)`) and the weights are bfloat16, the two
    projections become one matrix product over the concatenated hidden vectors:
    x + [o | g] [W_o | W_down]^T + (b_o + b_down), with the residual added on its 32-bit accumulator.

    Decode steps over few keys are bound by the latency of the attention kernels, not by memory: there the
    feed-forward runs whole on a second stream beside the mixer (its two products stream their weights
    while the attention kernels wait for theirs), and the mixer's output product - over its columns of
    the fused matrix - adds x and the feed-forward's result on its 32-bit accumulator."""
    norm_names = ("input",)

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        self.fused_weight = None
        import torch
        fusable = all(hasattr(p, "output_projection") and hasattr(p, "forward_hidden") for p in (self.mixer, self.ffn))
        if fusable and runtime.dtype == torch.bfloat16:
            (wm, bm), (wf, bf) = self.mixer.output_projection(), self.ffn.output_projection()
            if (wm.dtype == wf.dtype == torch.bfloat16 and wm.shape[0] == wf.shape[0]
                    and wm.shape[1] % 8 == 0 and wf.shape[1] % 8 == 0):
                self.k_mixer = wm.shape[1]
                self.fused_weight = torch.cat([wm, wf], dim=1).contiguous()
                biases = [b.float() for b in (bm, bf) if b is not None]
                self.fused_bias = sum(biases[1:], biases[0]) if biases else None
                # the parts keep views of the fused matrix, so the weights are held once
                self.mixer.w_out = self.fused_weight[:, :self.k_mixer]
                self.ffn.down = self.fused_weight[:, self.k_mixer:]
                # the feed-forward's two matrices, taken as equal in size; a mixer that does not say what a key
                # costs it never runs beside the feed-forward
                self.ffn_bytes = 2 * self.ffn.down.numel() * self.fused_weight.element_size()
                self.key_bytes = getattr(self.mixer, "cache_bytes_per_key", None)

    def forward(self, x, step, cache_id):
        h = self.norms["input"].forward(x)
        if self.fused_weight is None:
            a = self.mixer.forward(h, step, cache_id)
            return self.ffn.forward(h, step, residuals=(x, a))
        import torch
        from .linear import linear
        b = step.batch
        side = getattr(step, "side_stream", None)
        share = SIDE_BRANCH_SHARE if h.shape[0] <= SHARED_SM_ROWS else SIDE_BRANCH_SHARE_MANY_ROWS
        if (side is not None and b.decode and self.key_bytes is not None
                and h.shape[0] * (b.max_total or step.cache.max_context) * self.key_bytes <= share * self.ffn_bytes):
            from .linear import beside_main_stream, shared_sms
            # m is read on the main stream, so it comes from the main stream's memory; g lives on the second stream only
            m = torch.empty((h.shape[0], self.fused_weight.shape[0]), dtype=h.dtype, device=h.device)
            # the two streams' products side by side on every SM (up to 8 rows: +1 to +5 % tokens a second; 16 rows: -1 %)
            with shared_sms() if h.shape[0] <= SHARED_SM_ROWS else contextlib.nullcontext():
                with beside_main_stream(side, h.device) as beside:
                    g = self.ffn.forward_hidden(h, step)
                    linear(g, self.fused_weight[:, self.k_mixer:], self.fused_bias, out=m)
                o = self.mixer.forward_hidden(h, step, cache_id)
                beside.join()
                return linear(o, self.fused_weight[:, :self.k_mixer], None, residuals=(x, m))
        hidden = torch.empty((h.shape[0], self.fused_weight.shape[1]), dtype=h.dtype, device=h.device)
        self.mixer.forward_hidden(h, step, cache_id, out=hidden[:, :self.k_mixer])
        self.ffn.forward_hidden(h, step, out=hidden[:, self.k_mixer:])
        return linear(hidden, self.fused_weight, self.fused_bias, residuals=(x,))


class SequentialBlock(Arrangement):
    norm_names = ("input", "post_mixer")

    def forward(self, x, step, cache_id):
        x = self.mixer.forward(self.norms["input"].forward(x), step, cache_id, residuals=(x,))
        return self.ffn.forward(self.norms["post_mixer"].forward(x), step, residuals=(x,))


class PendingUpdate:
    """A branch that is still to be added to the 32-bit stream: x += mult * branch.  The layer that ends with it
    leaves it to the next layer's first norm, which adds it in the same kernel; whoever needs the stream itself
    (`StepContext.settle`) adds it with a kernel of its own."""

    def __init__(self, branch, mult):
        self.branch, self.mult = branch, mult

    def apply(self, x):
        from ..csrc import ops
        ops.rmsnorm(x, None, 0.0, update=self.branch, mult=self.mult, want_norm=False)
        return x


class ScaledResidualBlock(Arrangement):
    """x += m mixer(norm_1(x)); x += m ffn(norm_2(x)), with the residual stream x in 32-bit whatever the engine's
    type (the embedding delivers it so) and updated in place; a layer may have no feed-forward.  The branches'
    results arrive in 32-bit from their last product; the update x + m y and the norm that follows it are one
    kernel, also across layers: a layer leaves its last branch pending (`step.pending`) for the next layer's first
    norm.  Norms must offer `forward_update` (the RMS norm does)."""
    norm_names = ("input",)
    takes_pending = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        import inspect
        import torch
        if self.ffn is not None and "post_mixer" not in self.norms:
            raise QStreamError(QsError.INVALID_MODEL, "a scaled-residual layer with a feed-forward needs the norm 'post_mixer'")
        self.mult = float(spec.residual_scale)
        self.wide = torch.float32
        # parts of another make (a test's toy mixer) may not take `out_dtype`; their result is used as it comes
        self._typed = {id(p): "out_dtype" in inspect.signature(p.forward).parameters for p in (self.mixer, self.ffn) if p}

    @classmethod
    def part_specs(cls, spec):
        yield "mixer", spec.mixer
        if spec.ffn is not None:
            yield "feed_forward", spec.ffn
        for norm_spec in spec.norms.values():
            yield "norm", norm_spec

    @classmethod
    def build(cls, spec, make, runtime):
        parts = {"mixer": make("mixer", spec.mixer), "ffn": make("feed_forward", spec.ffn) if spec.ffn is not None else None,
                 "norms": {name: make("norm", ns) for name, ns in spec.norms.items()}}
        return cls(spec, parts, runtime)

    def _wide(self, part):
        return {"out_dtype": self.wide} if self._typed[id(part)] else {}

    def forward(self, x, step, cache_id):
        before, step.pending = step.pending, None
        norm = self.norms["input"]
        h = norm.forward_update(x, before.branch, before.mult) if before is not None else norm.forward(x)
        y = self.mixer.forward(h, step, cache_id, **self._wide(self.mixer))
        if self.ffn is not None:
            h = self.norms["post_mixer"].forward_update(x, y, self.mult)
            y = self.ffn.forward(h, step, **self._wide(self.ffn))
        step.pending = PendingUpdate(y, self.mult)
        return x


class PendingNormedUpdate:
    """A branch that is still to be normed and added to the stream: x += norm(branch) with `norm`'s weight."""

    def __init__(self, branch, norm):
        self.branch, self.norm = branch, norm

    def apply(self, x):
        return self.norm.add_normed(x, self.branch)


class SandwichBlock(Arrangement):
    """A norm before and after each sublayer: x += norm_1b(mixer(norm_1(x))); x += norm_2b(ffn(norm_2(x))), with the
    residual stream x in 32-bit whatever the engine's type and updated in place; a layer may have no feed-forward.
    The branches arrive in 32-bit from their last product.  The norm of a branch, its addition to x and the norm that
    follows are one kernel, also across layers: a layer leaves its last branch pending (`step.pending`) for the
    next layer's first norm.  Norms must offer `forward_update(x, branch, branch_norm)` and `add_normed`."""
    norm_names = ("input", "post_input")
    takes_pending = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        import inspect
        import torch
        if self.ffn is not None and not {"post_mixer", "post_ffn"} <= set(self.norms):
            raise QStreamError(QsError.INVALID_MODEL, "a sandwich layer with a feed-forward needs the norms 'post_mixer' and 'post_ffn'")
        self.wide = torch.float32
        self._typed = {id(p): "out_dtype" in inspect.signature(p.forward).parameters for p in (self.mixer, self.ffn) if p}

    part_specs = classmethod(ScaledResidualBlock.part_specs.__func__)      # a layer may lack its feed-forward here too
    build = classmethod(ScaledResidualBlock.build.__func__)

    def _wide(self, part):
        return {"out_dtype": self.wide} if self._typed[id(part)] else {}

    def forward(self, x, step, cache_id):
        before, step.pending = step.pending, None
        norm = self.norms["input"]
        if isinstance(before, PendingNormedUpdate):
            h = norm.forward_update(x, before.branch, before.norm)
        else:
            h = norm.forward(before.apply(x) if before is not None else x)
        y = self.mixer.forward(h, step, cache_id, **self._wide(self.mixer))
        last = self.norms["post_input"]
        if self.ffn is not None:
            h = self.norms["post_mixer"].forward_update(x, y, last)
            y = self.ffn.forward(h, step, **self._wide(self.ffn))
            last = self.norms["post_ffn"]
        step.pending = PendingNormedUpdate(y, last)
        return x


class PostNormBlock(Arrangement):
    """The sublayers read the stream itself and a norm meets their results only: x += norm_1(mixer(x));
    x += norm_2(ffn(x)), with the residual stream x in 32-bit whatever the engine's type and updated in place; a layer
    may have no feed-forward.  The branches arrive in 32-bit from their last product.  The norm of a branch, its
    addition to x and the copy of the new x in the engine's type that the next sublayer reads are one kernel, also
    across layers: a layer leaves its last branch pending (`step.pending`) for the next layer's read.  Norms must
    offer `read_update(x, branch, branch_norm)`, `read` and `add_normed` (the stream norm does)."""
    norm_names = ("post_input",)
    takes_pending = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        import inspect
        import torch
        if self.ffn is not None and "post_ffn" not in self.norms:
            raise QStreamError(QsError.INVALID_MODEL, "a post-norm layer with a feed-forward needs the norm 'post_ffn'")
        self.wide = torch.float32
        self._typed = {id(p): "out_dtype" in inspect.signature(p.forward).parameters for p in (self.mixer, self.ffn) if p}

    part_specs = classmethod(ScaledResidualBlock.part_specs.__func__)      # a layer may lack its feed-forward here too
    build = classmethod(ScaledResidualBlock.build.__func__)

    def _wide(self, part):
        return {"out_dtype": self.wide} if self._typed[id(part)] else {}

    def forward(self, x, step, cache_id):
        before, step.pending = step.pending, None
        last = self.norms["post_input"]
        if isinstance(before, PendingNormedUpdate):
            h = last.read_update(x, before.branch, before.norm)
        else:
            h = last.read(before.apply(x) if before is not None else x)
        y = self.mixer.forward(h, step, cache_id, **self._wide(self.mixer))
        if self.ffn is not None:
            h = last.read_update(x, y, last)
            y = self.ffn.forward(h, step, **self._wide(self.ffn))
            last = self.norms["post_ffn"]
        step.pending = PendingNormedUpdate(y, last)
        return x


class HyperConnection(Part):
    """The tensors with which one sublayer meets a residual stream kept in several copies: the weights of the read
    (`in`), of the write (`out`), the matrix that mixes the copies (`mix`, [from, to]) and the vector that scales the
    sublayer's result.  All are used in 32-bit."""
    role = "connection"
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        from ..weights.loader import TensorDecl
        S = spec.streams
        d = {}
        if spec.layer_scale:
            d["scale"] = TensorDecl((spec.width,), "norm_weight")
        if spec.mixing:
            # drawn at random, the copies are averaged (S = 2) and read and written with weights around one
            d.update({"in": TensorDecl((S,), "norm_weight"), "out": TensorDecl((S,), "norm_weight"),
                      "mix": TensorDecl((S, S), "fraction")})
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.streams, self.width = int(spec.streams), int(spec.width)
        self.scale = tensors["scale"].float().contiguous() if spec.layer_scale else None
        self.w_in = self.w_out = self.mix = None
        if spec.mixing:
            self.w_in, self.w_out = tensors["in"].float().contiguous(), tensors["out"].float().contiguous()
            self.mix = tensors["mix"].float().contiguous()


class PendingHyperWrite:
    """A sublayer's result (one branch, or two with a factor each) that has not yet come back into the copies of the
    stream; the next layer's first read takes it over, anyone else applies it with a kernel of its own."""

    def __init__(self, connection, branches):
        self.connection, self.branches = connection, branches

    def write_args(self):
        c = self.connection
        (c1, y1), (c2, y2) = (self.branches + [(1.0, None)])[:2]
        return dict(y=y1, y_scale=c1, y2=y2, y2_scale=c2, layer_scale=c.scale, mix=c.mix, out_weights=c.w_out)

    def apply(self, x):
        from ..csrc import ops
        c = self.connection
        ops.hyper_mix_norm(x, c.streams, c.width, **self.write_args())
        return x


class HyperBlock(Arrangement):
    """The residual stream in S copies side by side, 32-bit, [T, S * width], updated in place.  A sublayer reads
    u = sum_s in[s] x_s, normed, and its result y (times the layer's scale vector) comes back as
    x_t <- sum_s mix[s][t] x_s + out[t] y for all t at once.  The write of one sublayer, the read of the next and that
    read's RMS norm are one kernel, also across layers (`step.pending`).  The first layer spreads the embedding's
    output over the copies.  A mixer that offers `branches` (two mixers side by side) hands its results over one by
    one with their factors, and the write adds them up.  A layer may have no feed-forward.  With one copy and no
    mixing tensors this is the plain 32-bit residual stream with a scale vector per sublayer."""
    norm_names = ("input",)
    takes_pending = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        import inspect
        import torch
        self.connections = parts["connections"]
        if "mixer" not in self.connections or (self.ffn is not None and not {"ffn"} <= set(self.connections)):
            raise QStreamError(QsError.INVALID_MODEL, "a hyper layer needs a connection per sublayer ('mixer', 'ffn')")
        if self.ffn is not None and "post_mixer" not in self.norms:
            raise QStreamError(QsError.INVALID_MODEL, "a hyper layer with a feed-forward needs the norm 'post_mixer'")
        self.streams, self.width = self.connections["mixer"].streams, self.connections["mixer"].width
        self.wide = torch.float32
        self._typed = {id(p): "out_dtype" in inspect.signature(p.forward).parameters for p in (self.mixer, self.ffn) if p}
        self.captures_any_step = self.captures_any_step and all(c.captures_any_step for c in self.connections.values())

    @classmethod
    def part_specs(cls, spec):
        yield "mixer", spec.mixer
        if spec.ffn is not None:
            yield "feed_forward", spec.ffn
        for norm_spec in spec.norms.values():
            yield "norm", norm_spec
        for connection in spec.connections.values():
            yield "connection", connection

    @classmethod
    def build(cls, spec, make, runtime):
        parts = {"mixer": make("mixer", spec.mixer), "ffn": make("feed_forward", spec.ffn) if spec.ffn is not None else None,
                 "norms": {name: make("norm", ns) for name, ns in spec.norms.items()},
                 "connections": {name: make("connection", cs) for name, cs in spec.connections.items()}}
        return cls(spec, parts, runtime)

    def cached_parts(self):
        return getattr(self.mixer, "cached_parts", lambda: [self.mixer])()

    def _read(self, x, connection, norm, before):
        """The normed input of a sublayer; `before`: a write that is still pending, done in the same pass."""
        from ..csrc import ops
        write = before.write_args() if before is not None else {}
        return ops.hyper_mix_norm(x, self.streams, self.width, in_weights=connection.w_in, norm_weight=norm.weight,
                                  offset=norm.offset, eps=norm.eps, out_dtype=self.runtime.dtype, **write)

    def forward(self, x, step, cache_id):
        from ..csrc import ops
        before, step.pending = step.pending, None
        if before is not None and not isinstance(before, PendingHyperWrite):
            x, before = before.apply(x), None
        if x.shape[1] != self.streams * self.width or x.dtype != self.wide:     # the embedding's output: every copy starts as it
            x = ops.hyper_spread(x if x.dtype == self.wide else ops.convert(x, self.wide), self.streams)
        h = self._read(x, self.connections["mixer"], self.norms["input"], before)
        if hasattr(self.mixer, "branches"):
            ys = self.mixer.branches(h, step, cache_id, out_dtype=self.wide)
        else:
            wide = {"out_dtype": self.wide} if self._typed[id(self.mixer)] else {}
            ys = [(1.0, self.mixer.forward(h, step, cache_id, **wide))]
        last = PendingHyperWrite(self.connections["mixer"], ys)
        if self.ffn is not None:
            h = self._read(x, self.connections["ffn"], self.norms["post_mixer"], last)
            wide = {"out_dtype": self.wide} if self._typed[id(self.ffn)] else {}
            last = PendingHyperWrite(self.connections["ffn"], [(1.0, self.ffn.forward(h, step, **wide))])
        step.pending = last
        return x


register("arrangement", "hyper", HyperBlock)
register("connection", "hyper_connection", HyperConnection)
register("arrangement", "parallel", ParallelBlock)
register("arrangement", "post_norm", PostNormBlock)
register("arrangement", "sandwich", SandwichBlock)
register("arrangement", "sequential", SequentialBlock)
register("arrangement", "scaled_residual", ScaledResidualBlock)


def build_block(spec, tensors_of, runtime):
    """Build one layer from its `BlockSpec`.  `tensors_of(part_spec, declaration)` returns
    the part's tensors by the part's own names."""
    def make(role, part_spec):
        cls = part_class(role, part_spec.kind)
        return cls(part_spec, tensors_of(part_spec, cls.declare(part_spec)), runtime)

    return part_class("arrangement", spec.arrangement).build(spec, make, runtime)
