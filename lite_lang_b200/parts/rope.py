"""Rotary position encoding with half-split pairs (i, i + d/2).

angle[p, i] = p * theta^(-2i/d); o[i] = x[i] cos - x[i+d/2] sin;
o[i+d/2] = x[i] sin + x[i+d/2] cos  (``litelang/kernel/develop_rope/rope.py:225-234``,
table ``litelang/models/qwen2/layer/pre_layer.py:21-30``).  The reference fixes
theta at 1e6 and casts the tables to half precision; here theta and the table
length come from the configuration and the table stays float32.

The table is built on the host with float32 operations in a fixed order, so the
angles are the same numbers on both precisions' paths.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from .base import PositionEncoding, register_part


def rope_table(rot_dim: int, theta: float, max_positions: int) -> torch.Tensor:
    """float32 [max_positions, rot_dim]: cos of the angles, then sin of the angles."""
    freqs = 1.0 / theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim)
    angle = torch.arange(0, max_positions, dtype=torch.float32)[:, None] * freqs[None, :]
    return torch.cat((torch.cos(angle), torch.sin(angle)), dim=1).contiguous()


class RotaryHalfSplit(PositionEncoding):
    fuses_with_store = True

    def __init__(self, spec):
        super().__init__(spec)
        self.rot_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rot_dim % 2:
            raise ValueError(f"rotary_dim {self.rot_dim} must be even")
        self.table: Optional[torch.Tensor] = None

    _shared = {}

    def prepare(self, device) -> None:
        key = (self.rot_dim, self.theta, self.max_positions, str(device))
        tab = RotaryHalfSplit._shared.get(key)
        if tab is None:
            tab = rope_table(self.rot_dim, self.theta, self.max_positions).to(device)
            RotaryHalfSplit._shared[key] = tab
        self.table = tab

    def fused_table(self) -> torch.Tensor:
        return self.table

    def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim, num_tokens) -> None:
        ops.bias_rope_store(qkv, None, positions, self.table, num_heads, num_kv_heads, head_dim,
                            None, None, None, 1, None, num_tokens)


class RotaryComputed(PositionEncoding):
    """Rotary encoding whose angles are made in the kernel: angle = float32(position) * f_i with
    f_i = theta^(-2i/rotary_dim) / ``position_scale`` (linear scaling of the positions; 1: none), computed in
    float64 on the host and rounded to float32 once.  No table, so no limit on the positions.  ``layout``:
    "interleaved" pairs channel 2i with 2i+1, "half_split" pairs i with i + rotary_dim/2; channels from
    ``rotary_dim`` on are left as they are.  (u, v) -> (u cos a - v sin a, v cos a + u sin a).

    ``scaling`` (optional: ``factor``, ``original``, ``fast``, ``slow``) stretches the slow frequencies only, so
    that a model trained on ``original`` positions reaches ``factor`` times as far (YaRN): with
    d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), lo = max(floor d(fast), 0), hi = min(ceil d(slow),
    rotary_dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    f_i / factor * r_i + f_i (1 - r_i); cos and sin are both multiplied by ``amplitude`` = 0.1 ln(factor) + 1
    (an attention that uses this part reads it and hands it to its kernel)."""

    computed = True
    fuses_with_store = False

    def __init__(self, spec):
        super().__init__(spec)
        self.rot_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.position_scale = float(spec.params.get("position_scale", 1.0))
        layout = str(spec.params.get("layout", "interleaved"))
        if layout not in ("interleaved", "half_split"):
            raise ValueError(f"rope_computed: layout {layout!r} is neither 'interleaved' nor 'half_split'")
        if self.rot_dim % 2 or self.rot_dim < 0 or self.position_scale <= 0:
            raise ValueError("rope_computed: rotary_dim must be even and position_scale positive")
        self.interleaved = layout == "interleaved"
        self.freq: Optional[torch.Tensor] = None
        self.amplitude = 1.0
        sc = spec.params.get("scaling")
        self.scaling = None
        if sc:
            self.scaling = {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")}
            if self.scaling["factor"] <= 0 or self.scaling["original"] <= 0 or self.theta <= 1.0:
                raise ValueError("rope_computed: scaling needs a positive factor and original length, theta above 1")
            self.amplitude = 0.1 * math.log(self.scaling["factor"]) + 1.0

    def frequencies(self) -> torch.Tensor:
        """float64 [rotary_dim / 2]: what a position is multiplied by for each pair."""
        i = torch.arange(0, self.rot_dim // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(self.rot_dim, 1))
        f = f / self.position_scale
        if self.scaling is not None:
            sc = self.scaling

            def turns(t: float) -> float:
                return self.rot_dim * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turns(sc["fast"])), 0)
            hi = min(math.ceil(turns(sc["slow"])), self.rot_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        return f

    def prepare(self, device) -> None:
        self.freq = self.frequencies().to(torch.float32).to(device).contiguous() if self.rot_dim else None

    def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim, num_tokens) -> None:
        if self.amplitude != 1.0:
            raise ValueError("rope_computed: a scaled rotation's amplitude is applied by the attention part that "
                             "names it (modulated_attention)")
        ops.bias_rotate_store(qkv[:num_tokens], None, positions, self.freq, self.interleaved, num_heads, num_kv_heads,
                              head_dim, head_dim, None, None, None, 1, None)


register_part("position", "rope_half_split", RotaryHalfSplit)
register_part("position", "rope_computed", RotaryComputed)
