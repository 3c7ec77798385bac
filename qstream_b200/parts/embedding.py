"""Token embeddings: the plain table x[t] = table[token[t]], no position term, no scale (QStream
src/engine.c:710-765), and a scaled table with a second, hashed table of token pairs."""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Embedding, register


class TokenEmbedding(Embedding):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.vocab_size, spec.width))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]

    def forward(self, step):
        return ops.embedding(self.weight, step.batch.tokens, self.runtime.dtype)


class PairEmbedding(Embedding):
    """x = table[token] * scale + pair[hash(previous token, token)]: a second table indexed by a hash of the
    token and the one before it (its last row for a sequence's first token).  The previous token of a sequence
    whose earlier tokens came in earlier steps is state: one int32 per slot, kept after every step.  The
    result may be wider than the engine's type (a 32-bit residual stream)."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"weight": TensorDecl((spec.vocab_size, spec.width))}
        if spec.buckets:
            d["pair"] = TensorDecl((spec.buckets + 1, spec.width))
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        import torch
        self.weight = tensors["weight"]
        self.pair = tensors["pair"] if spec.buckets else None
        self.out_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, None: runtime.dtype}[spec.stream_dtype]

    def state_need(self):
        import torch
        from ..cache import StateNeed
        return StateNeed((1,), torch.int32) if self.pair is not None else None

    def forward(self, step):
        b, s = step.batch, self.spec
        last = step.state("embedding") if self.pair is not None else None
        x = ops.embedding_hashed(self.weight, self.pair, s.scale, s.buckets, s.mul_prev, s.mul_cur, b.tokens,
                                 b.tok_slot, b.tok_pos, last, self.out_dtype)
        if last is not None:        # after the lookup has read it: the token each sequence ends this step with
            ops.keep_last_rows(last, b.tokens.view(-1, 1), b.seq_start, b.seq_slot, b.n_seq)
        return x


class NormedEmbedding(Embedding):
    """x = norm(table[token]) with a weight and no bias, delivered in the stream's type (which may be wider than the
    engine's)."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.vocab_size, spec.width)),
                "norm": TensorDecl((spec.width,), "norm_delta" if getattr(spec, "offset", 0.0) else "norm_weight")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        import torch
        self.weight, self.norm = tensors["weight"], tensors["norm"]
        self.out_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, None: runtime.dtype}[spec.stream_dtype]

    def forward(self, step):
        b, s = step.batch, self.spec
        x = ops.embedding_hashed(self.weight, None, 1.0, 0, 0, 0, b.tokens, b.tok_slot, b.tok_pos, None, self.out_dtype)
        if getattr(s, "offset", 0.0) and not s.center:      # a weight stored around zero: the RMS norm with its offset
            return ops.rmsnorm(x, self.norm, s.eps, s.offset, out_dtype=self.out_dtype)
        return ops.branch_norm(x, self.norm, s.eps, s.center, in_place=True)


register("embedding", "embedding", TokenEmbedding)
register("embedding", "normed_embedding", NormedEmbedding)
register("embedding", "pair_embedding", PairEmbedding)
