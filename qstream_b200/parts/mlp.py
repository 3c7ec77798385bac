"""Dense feed-forward: up projection + bias, activation, down projection + bias
(QStream src/engine.c:1150-1170; the activation's tanh form src/kernels_scalar.c:135-142,
the erf form is GPT-J's 'gelu').  The activation runs on the 32-bit accumulator of the
up projection; residuals are added on the accumulator of the down projection."""
from __future__ import annotations

from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import FeedForward, register
from .linear import linear


class Mlp(FeedForward):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"up": TensorDecl((spec.inner, spec.width)), "down": TensorDecl((spec.width, spec.inner))}
        if spec.bias:
            d["up_bias"] = TensorDecl((spec.inner,), "bias")
            d["down_bias"] = TensorDecl((spec.width,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.activation not in ops.ACTIVATIONS:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"activation '{spec.activation}' has no kernel")
        self.up, self.down = tensors["up"], tensors["down"]
        self.up_bias = tensors.get("up_bias") if spec.bias else None
        self.down_bias = tensors.get("down_bias") if spec.bias else None

    def forward(self, h, step, residuals=(), out_dtype=None):
        g = self.forward_hidden(h, step)
        return linear(g, self.down, self.down_bias, residuals=residuals, out_dtype=out_dtype)

    # See Attention.output_projection: the same pair for a parallel block that fuses both projections.
    def output_projection(self):
        return self.down, self.down_bias

    def forward_hidden(self, h, step, out=None):
        """The activated up projection: [T, inner], written to `out` if given."""
        return linear(h, self.up, self.up_bias, activation=self.spec.activation, out=out)


class GatedMlp(FeedForward):
    """down(act(gate h) * (up h)), no biases: gate and up are one product over the stacked weights, the
    activation and the product of the halves one kernel in 32-bit (the reference's llama feed-forward,
    QStream src/engine.c:1115-1148)."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"gate": TensorDecl((spec.inner, spec.width)), "up": TensorDecl((spec.inner, spec.width)),
             "down": TensorDecl((spec.width, spec.inner))}
        if getattr(spec, "bias", False):
            d.update({"gate_bias": TensorDecl((spec.inner,), "bias"), "up_bias": TensorDecl((spec.inner,), "bias"),
                      "down_bias": TensorDecl((spec.width,), "bias")})
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        import torch
        if spec.activation not in ops.ACTIVATIONS:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"activation '{spec.activation}' has no kernel")
        self.gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down = tensors["down"]
        self.gate_up_bias = self.down_bias = None
        if getattr(spec, "bias", False):
            self.gate_up_bias = torch.cat([tensors["gate_bias"].float(), tensors["up_bias"].float()]).contiguous()
            self.down_bias = tensors["down_bias"]

    def forward(self, h, step, residuals=(), out_dtype=None):
        g = ops.gated_act(linear(h, self.gate_up, self.gate_up_bias), self.spec.activation)
        return linear(g, self.down, self.down_bias, residuals=residuals, out_dtype=out_dtype)


# A step of single tokens, or of at most this many rows, lets every (token, expert) pair find its expert's matrices
# on the device (such a step can be captured and replayed); a larger one orders the pairs by expert and runs one
# product per expert.
INDIRECT_ROWS = 32


class RoutedExperts(FeedForward):
    """A mixture of small feed-forward layers W_down act(W_up h): a router picks `top` experts per token among the
    experts of the best groups (csrc/moe.cu), their outputs are added with the router's weights in 32-bit, and an
    optional shared expert runs for every token, multiplied by a sigmoid gate of its own.  The router's logits are
    a product with 32-bit sums and a 32-bit result; the shared gate's row rides in the same product.  Options of the
    spec: softmax scores, a group's score as its largest, no correction, an ungated shared expert, and gated experts
    (an expert's gate rows stacked above its up rows in one matrix; the clamped gated unit is a kernel of its own
    between the two products)."""
    captures_any_step = False           # a step with many tokens reads the experts' row counts on the host

    @classmethod
    def declare(cls, spec):
        d = {"router": TensorDecl((spec.n_experts, spec.width))}
        gated = getattr(spec, "gated", False)
        if getattr(spec, "correction", True):
            d["correction"] = TensorDecl((spec.n_experts,), "bias")
        for e in range(spec.n_experts):
            d[f"up{e}"], d[f"down{e}"] = TensorDecl((spec.inner, spec.width)), TensorDecl((spec.width, spec.inner))
            if gated:
                d[f"gate{e}"] = TensorDecl((spec.inner, spec.width))
        if spec.shared_inner:
            d.update({"shared_up": TensorDecl((spec.shared_inner, spec.width)),
                      "shared_down": TensorDecl((spec.width, spec.shared_inner))})
            if getattr(spec, "shared_gate", True):
                d["shared_gate"] = TensorDecl((1, spec.width))
            if gated:
                d["shared_gate_proj"] = TensorDecl((spec.shared_inner, spec.width))
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        import torch
        if spec.activation not in ops.ACTIVATIONS:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"activation '{spec.activation}' has no kernel")
        E = spec.n_experts
        self.gated = bool(getattr(spec, "gated", False))
        self.scores, self.group_score = getattr(spec, "scores", "sigmoid"), getattr(spec, "group_score", "top2")
        if self.scores not in ("sigmoid", "softmax") or self.group_score not in ("top2", "max"):
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"routed experts: scores '{self.scores}', group score '{self.group_score}'")
        # (limit, alpha, shift) of the clamped gated unit, for the routed experts and for the shared one
        self.glu = (float(spec.limit), float(spec.glu_alpha), float(spec.glu_shift)) if self.gated else None
        self.shared_glu = (float(spec.shared_limit), float(spec.glu_alpha), float(spec.glu_shift)) if self.gated else None
        if self.gated:                                  # an expert's gate rows above its up rows: one product for both
            self.w_up = torch.stack([torch.cat([tensors[f"gate{e}"], tensors[f"up{e}"]], dim=0) for e in range(E)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[f"up{e}"] for e in range(E)]).contiguous()      # [E, inner, width]
        self.w_down = torch.stack([tensors[f"down{e}"] for e in range(E)]).contiguous()      # [E, width, inner]
        self.correction = tensors["correction"].float().contiguous() if getattr(spec, "correction", True) else None
        self.shared = bool(spec.shared_inner)
        self.shared_gate = self.shared and bool(getattr(spec, "shared_gate", True))
        rows = [tensors["router"]] + ([tensors["shared_gate"]] if self.shared_gate else [])
        self.w_router = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0]
        if self.shared:
            self.shared_up, self.shared_down = tensors["shared_up"], tensors["shared_down"]
            if self.gated:
                self.shared_up = torch.cat([tensors["shared_gate_proj"], tensors["shared_up"]], dim=0).contiguous()

    def forward(self, h, step, residuals=(), out_dtype=None):
        import torch
        s, b = self.spec, step.batch
        z = linear(h, self.w_router, out_dtype=torch.float32)
        idx, wts, gate = ops.moe_route(z, self.correction, s.n_experts, s.top, s.groups, s.keep, s.route_scale,
                                       gate_col=s.n_experts if self.shared_gate else -1, scores=self.scores,
                                       group_score=self.group_score)
        shared = None
        if self.shared and self.gated:
            shared = linear(ops.clamped_glu(linear(h, self.shared_up), *self.shared_glu), self.shared_down, out_dtype=torch.float32)
        elif self.shared:
            shared = linear(linear(h, self.shared_up, activation=s.activation), self.shared_down, out_dtype=torch.float32)
        if b.decode or h.shape[0] <= INDIRECT_ROWS:
            out = ops.moe_experts_indirect(h, self.w_up, self.w_down, idx, wts, b.tok_slot, s.activation, shared, gate, glu=self.glu)
        else:
            offsets, place_token, pair_place = ops.moe_sort(idx, s.n_experts)
            rows = ops.gather_rows(h, place_token)
            hidden = torch.empty((rows.shape[0], self.w_up.shape[1]), dtype=h.dtype, device=h.device)
            y = torch.empty((rows.shape[0], s.width), dtype=torch.float32, device=h.device)
            bounds = offsets.tolist()                   # waits for the device: how many rows each expert got
            ops.expert_products(hidden, rows, self.w_up, bounds)        # a product per expert, launched by one call
            if self.gated:
                hidden = ops.clamped_glu(hidden, *self.glu)             # one launch for all experts' rows
            else:
                ops.activate(hidden, s.activation)
            ops.expert_products(y, hidden, self.w_down, bounds)
            out = ops.moe_combine(y, pair_place, wts, b.tok_slot, shared, gate)
        if residuals:
            raise QStreamError(QsError.INVALID_INPUT, "routed experts: residuals are added by the arrangement")
        return out if out_dtype in (None, torch.float32) else ops.convert(out, out_dtype)


register("feed_forward", "mlp", Mlp)
register("feed_forward", "gated_mlp", GatedMlp)
register("feed_forward", "routed_experts", RoutedExperts)
