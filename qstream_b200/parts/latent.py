"""Attention through a cached latent: per token the cache keeps one normed latent vector c and one rotated key part
shared by all heads; a head's unrotated key is W_uk c and its value W_uv c.

The key map is folded into the query, q' = W_uk^T q_unrotated, so that a head's score is q' . c + q_rot . k_rot and
its output W_uv (sum_j p_j c_j): attention with one key head of size kv_rank + rot_dim whose values are the keys'
first kv_rank elements.  That form runs on the library's own attention kernels (decode, prefill, generic) through
the paged cache, with keys [c | k_rot] and values c; a layer that shares another's cache reads that entry with its
own W_uk and W_uv.  Norms, rotation, scores and softmax are 32-bit; the projections run in the engine's type.
Options of the spec: a learned sink per head in the softmax's denominator; a sigmoid gate per head from the mixer's
input, whose rows ride in the down projections' product; the rotation's pairing (halves or neighbours) is the
position part's.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

from ..cache import KvNeed
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .attention import attend
from .base import Mixer, part_class, register
from .linear import linear


FEW_TOKENS = 64         # up to here the per-head maps of a step run as one launch on the CUDA cores


class LatentAttention(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        H, dq = spec.n_heads, spec.head_dim + spec.rot_dim
        d = {"dq": TensorDecl((spec.q_rank, spec.width)), "dq_norm": TensorDecl((spec.q_rank,), "norm_weight"),
             "uq": TensorDecl((H * dq, spec.q_rank)), "uk": TensorDecl((H * spec.head_dim, spec.kv_rank)),
             "uv": TensorDecl((H * spec.v_head_dim, spec.kv_rank)), "o": TensorDecl((spec.width, H * spec.v_head_dim))}
        if not spec.shares_cache:
            d["dkv"] = TensorDecl((spec.kv_rank + spec.rot_dim, spec.width))
            d["dkv_norm"] = TensorDecl((spec.kv_rank,), "norm_weight")
        if getattr(spec, "sink", False):
            d["sink"] = TensorDecl((H,), "bias")
        if getattr(spec, "head_gate", False):
            d["g"] = TensorDecl((H, spec.width))
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.position is None:
            raise QStreamError(QsError.INVALID_MODEL, "latent attention needs a rotation for its shared key part")
        self.position = part_class("position", spec.position.kind)(spec.position, {}, runtime)
        if not hasattr(self.position, "frequencies") or self.position.rotary_dim > spec.rot_dim:
            raise QStreamError(QsError.INVALID_MODEL, "latent attention: the rotation must give frequencies for at most rot_dim dims")
        if spec.kv_rank > 512 or spec.kv_rank + spec.rot_dim > 2048:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"latent attention: a latent of {spec.kv_rank} (+ {spec.rot_dim}) exceeds the attention kernels")
        H, dn, r = spec.n_heads, spec.head_dim, spec.kv_rank
        # both down projections read h: one product
        self.head_gate = bool(getattr(spec, "head_gate", False))
        self.sink = tensors["sink"].float().contiguous() if getattr(spec, "sink", False) else None
        self.interleaved = getattr(spec.position, "layout", "half") == "interleaved"
        down = [tensors["dq"]] + ([] if spec.shares_cache else [tensors["dkv"]]) + ([tensors["g"]] if self.head_gate else [])
        self.w_down = torch.cat(down, dim=0).contiguous() if len(down) > 1 else down[0]
        self.q_norm = tensors["dq_norm"]
        self.kv_norm = None if spec.shares_cache else tensors["dkv_norm"]
        self.w_uq = tensors["uq"]
        # head h's key map as the matrix of the folded product: [kv_rank, head_dim] = W_uk[h]^T
        self.w_uk_t = tensors["uk"].view(H, dn, r).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"]
        self.w_uv_heads = self.w_uv.view(H, spec.v_head_dim, r)          # the same memory, head by head
        self.w_out = tensors["o"]
        # what the attention kernels see: one key head of kv_rank + rot_dim, values of kv_rank
        self.as_attention = SimpleNamespace(n_heads=H, n_kv_heads=1, head_dim=r + spec.rot_dim, value_dim=r,
                                            scale=float(spec.score_scale), window=0, softcap=0.0)

    @property
    def cache_bytes_per_key(self) -> int:
        return (2 * self.spec.kv_rank + self.spec.rot_dim) * self.w_uq.element_size()

    def kv_need(self):
        if self.spec.shares_cache:
            return None
        s = self.spec
        return KvNeed(n_kv_heads=1, head_dim=s.kv_rank + s.rot_dim, window=0, v_head_dim=s.kv_rank)

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b, pos = self.spec, step.batch, self.position
        view = step.kv(cache_id)
        H, dn, dr, dv, r = s.n_heads, s.head_dim, s.rot_dim, s.v_head_dim, s.kv_rank
        d = linear(h, self.w_down)
        cq = ops.latent_prepare(d[:, :s.q_rank], self.q_norm, s.q_rank, None if s.shares_cache else d[:, s.q_rank:s.q_rank + r + dr],
                                self.kv_norm, r, dr, pos.rotary_dim, pos.frequencies, pos.magnitude, s.eps, b.tok_slot,
                                b.tok_pos, view.page_table, view.page_tokens, view.k, view.v, step.status,
                                interleaved=self.interleaved)
        q = linear(cq, self.w_uq)
        T = q.shape[0]
        q_abs = torch.empty((T, H * (r + dr)), dtype=q.dtype, device=q.device)
        ops.latent_q_rotate(q_abs, q, H, dn, dr, r, pos.rotary_dim, pos.frequencies, pos.magnitude, b.tok_slot, b.tok_pos,
                            interleaved=self.interleaved)
        few = T <= FEW_TOKENS                   # one launch for all heads; else a product per head, dealt to several streams
        (ops.head_linear if few else ops.head_products)(q_abs, q, self.w_uk_t, H)
        latent = attend(q_abs, self.as_attention, step, view, sink=self.sink)
        o = torch.empty((T, H * dv), dtype=q.dtype, device=q.device)
        (ops.head_linear if few else ops.head_products)(o, latent, self.w_uv_heads, H)
        if self.head_gate:                              # one gate value per head, the product's last H columns
            o = ops.gated_group_norm(o, 0, None, d[:, d.shape[1] - H:], "sigmoid", 0.0, o.dtype, gate_span=dv)
        return linear(o, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


register("mixer", "latent_attention", LatentAttention)
