"""Rotary position encoding on the first `rotary_dim` dims of each head, pairs (i, i+1).

theta(pos, i) = pos * base^(-i / rotary_dim), i = 0, 2, ...; (a, b) -> (a cos - b sin,
a sin + b cos): QStream src/engine.c:205-234, which rotates the whole head; here the
rotated width is a parameter.  The angles are computed in float64 and the table
[max_positions, rotary_dim/2, (cos, sin)] is kept in float32.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import PositionEncoding, register


_TABLES: dict = {}      # layers with the same rotation share one table


def _table(rotary_dim: int, base: float, max_positions: int, device):
    key = (rotary_dim, float(base), int(max_positions), str(device))
    if key not in _TABLES:
        i = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -i / max(rotary_dim, 1))
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * freq[None, :]
        _TABLES[key] = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous().to(device)
    return _TABLES[key]


class RotaryInterleaved(PositionEncoding):
    captures_any_step = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec.rotary_dim)
        # Attention fuses the rotation with its cache write when a position part offers this.
        self.fused_table = _table(self.rotary_dim, spec.base, spec.max_positions, runtime.device) if self.rotary_dim > 0 else None

    def apply(self, q, k, step, n_heads, n_kv_heads, head_dim):
        """Rotate q and k in place (no cache write); for mixers that do not fuse the rotation with
        their cache write.  A rotary width of 0 rotates nothing."""
        if self.fused_table is None:
            return
        b = step.batch
        for x, heads in ((q, n_heads), (k, n_kv_heads)):
            if x is not None and heads > 0:
                ops.rope_store(x, None, None, heads, 0, head_dim, self.rotary_dim, self.fused_table,
                               b.tok_slot, b.tok_pos, None, 64, None, None, step.status, settled=True)


class RotaryHalfTable(PositionEncoding):
    """Element i of the first `rotary_dim` dims of each head is paired with element i + rotary_dim / 2, angle
    position * base^(-2i / rotary_dim): the angles of the interleaved form, so the two share their tables; the kernel
    is told which elements make a pair.  Attention fuses the rotation with its cache write."""
    captures_any_step = True
    half_layout = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec.rotary_dim)
        self.fused_table = _table(self.rotary_dim, spec.base, spec.max_positions, runtime.device) if self.rotary_dim > 0 else None

    def apply(self, q, k, step, n_heads, n_kv_heads, head_dim):
        """Rotate q and k in place (no cache write), in their own type."""
        if self.fused_table is None:
            return
        b = step.batch
        for x, heads in ((q, n_heads), (k, n_kv_heads)):
            if x is not None and heads > 0:
                ops.rope_store(x, None, None, heads, 0, head_dim, self.rotary_dim, self.fused_table,
                               b.tok_slot, b.tok_pos, None, 64, None, None, step.status, settled=True, half_layout=True)


def scaled_frequencies(rotary_dim: int, base: float, scaling=None):
    """The rotary_dim / 2 frequencies base^(-2i / rotary_dim) in float64, rescaled in the YaRN manner if `scaling`
    (factor, original, fast, slow) is given, and the factor on cos and sin (1 without scaling)."""
    import math
    half = rotary_dim // 2
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / max(rotary_dim, 1))
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):      # the dimension whose wavelength fits `turns` times into the original context
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), rotary_dim - 1)
    ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class RotaryHalf(PositionEncoding):
    """Element i of the first `rotary_dim` dims is paired with element i + rotary_dim / 2.  The part holds the
    frequencies (float64, on the device) and the factor on cos and sin; the kernels that rotate take the angle as
    position * frequency, so no table of positions is kept."""
    captures_any_step = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec.rotary_dim)
        f, self.magnitude = scaled_frequencies(self.rotary_dim, spec.base, spec.scaling)
        self.frequencies = f.contiguous().to(runtime.device)


register("position", "rotary_interleaved", RotaryInterleaved)
register("position", "rotary_half", RotaryHalf)
register("position", "rotary_half_table", RotaryHalfTable)
