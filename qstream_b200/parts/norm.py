"""LayerNorm with weight and optional bias (QStream src/kernels_scalar.c:151-171), and the RMS norm
x / sqrt(mean(x^2) + eps) * (offset + weight) (the reference's `rmsnorm`, src/kernels_scalar.c:173-186, has
offset 0; weights stored around zero take offset 1)."""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Norm, register


class LayerNorm(Norm):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"weight": TensorDecl((spec.size,), "norm_weight")}
        if spec.bias:
            d["bias"] = TensorDecl((spec.size,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias") if spec.bias else None
        self.eps = float(spec.eps)

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps, settled=True)     # a model's weights are old


class RmsNorm(Norm):
    """Reads x in its own type (a 32-bit residual stream in a bfloat16 engine, for instance) and writes the
    engine's type.  `forward_update` first adds a scaled branch to x, in place, in the same kernel."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.size,), "norm_delta" if spec.offset else "norm_weight")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]
        self.eps, self.offset = float(spec.eps), float(spec.offset)

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps, self.offset, out_dtype=self.runtime.dtype)

    def forward_update(self, x, branch, mult):
        """x <- x + mult * branch (in place), then the norm of the new x."""
        return ops.rmsnorm(x, self.weight, self.eps, self.offset, out_dtype=self.runtime.dtype, update=branch, mult=mult)


class StreamNorm(Norm):
    """A norm with a weight and no bias (layer norm if the spec says `center`, else RMS) that reads the stream in its
    own type and writes the engine's.  `forward_update` first adds a branch to x, in place, in the same kernel; the
    branch may itself be normed with another such norm's weight (`branch_norm`)."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.size,), "norm_weight")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]
        self.eps, self.center = float(spec.eps), bool(spec.center)

    def forward(self, x):
        return ops.branch_norm(x, self.weight, self.eps, self.center, out_dtype=self.runtime.dtype)

    def forward_update(self, x, branch, branch_norm=None):
        """x <- x + branch_norm(branch) (in place; the plain sum without `branch_norm`), then the norm of the new x."""
        return ops.branch_norm(x, self.weight, self.eps, self.center, out_dtype=self.runtime.dtype, branch=branch,
                               branch_weight=branch_norm.weight if branch_norm is not None else None)

    def add_normed(self, x, branch):
        """x <- x + norm(branch) * weight, in place: this norm applied to a branch on its way into the stream."""
        ops.branch_norm(x, None, self.eps, self.center, branch=branch, branch_weight=self.weight, want_norm=False)
        return x

    def read(self, x):
        """The stream as a sublayer without a norm of its own reads it: x in the engine's type (x itself where that is
        the stream's type; nobody changes x while the sublayer runs)."""
        if x.dtype == self.runtime.dtype:
            return x
        return ops.branch_norm(x, None, self.eps, self.center, out_dtype=self.runtime.dtype)

    def read_update(self, x, branch, branch_norm):
        """x <- x + branch_norm(branch) (in place), then `read` of the new x, in one kernel."""
        if x.dtype == self.runtime.dtype:
            return branch_norm.add_normed(x, branch)
        return ops.branch_norm(x, None, self.eps, self.center, out_dtype=self.runtime.dtype, branch=branch,
                               branch_weight=branch_norm.weight)


class StreamSumNorm(Norm):
    """The RMS norm of the sum of a residual stream's copies: rows [n, streams * size] in 32-bit, the copies side by
    side; the result [n, size] in the engine's type."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.size,), "norm_delta" if spec.offset else "norm_weight")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]
        self.eps, self.offset = float(spec.eps), float(spec.offset)

    def forward(self, x):
        s = self.spec
        return ops.hyper_mix_norm(x, s.streams, s.size, norm_weight=self.weight, offset=self.offset, eps=self.eps,
                                  out_dtype=self.runtime.dtype)


register("norm", "layernorm", LayerNorm)
register("norm", "stream_sum_rmsnorm", StreamSumNorm)
register("norm", "stream_norm", StreamNorm)
register("norm", "rmsnorm", RmsNorm)
