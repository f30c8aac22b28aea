"""Two mixers side by side: both read the same input, and their outputs are joined.

``left`` and ``right`` are ordinary mixer parts (each given as {"kind": ..., "params": ...}; their tensors live
under ``left.`` and ``right.`` of this part's prefix, and each owns its memory in the cache manager: pages for
one, a state record for the other, whatever they ask for).  The join is

    out = (rms(left(x)) * w_left + rms(right(x)) * w_right) / 2

with RMS norms over the model width (x / sqrt(mean(x^2) + eps), plain weights ``left.out`` and ``right.out``).
A bias on the left mixer's output projection is added inside the join's pass instead of in one of its own.

``join`` = "sum" is the plain weighted sum instead: out = ``left_scale`` * left(x) + ``right_scale`` * right(x),
without norms or tensors of its own.  Both members then end in a projection without a bias, so the join is one
product: each member writes what its projection would read, times its constant (before that value's one
rounding), into its columns of one buffer, and the buffer is multiplied by the two projections' matrices side
by side, [W_left | W_right].  Members take part through ``inner_width``, ``inner_weight()`` and
``forward_inner(x, step, cache, out, out_scale)``.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, TensorDecl, build_part, register_part, whole_output

_SIDES = ("left", "right")


class SideBySide(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.eps = float(p.get("eps", 0.0))
        self.join = str(p.get("join", "rms_mean"))
        if self.join not in ("rms_mean", "sum"):
            raise ValueError(f"side_by_side: join {self.join!r}; built: rms_mean, sum")
        self.scales = {"left": float(p.get("left_scale", 1.0)), "right": float(p.get("right_scale", 1.0))}
        self.sides: Dict[str, Mixer] = {}
        for side in _SIDES:
            sub = p[side]
            m = build_part("mixer", PartSpec(str(sub["kind"]), dict(sub["params"]), self.prefix + side + "."))
            m.partial_ok = False
            self.sides[side] = m
        self.left, self.right = self.sides["left"], self.sides["right"]
        if hasattr(self.left, "defer_out_bias"):
            self.left.defer_out_bias = True     # added in the join
        self.w_left = self.w_right = None
        self.w_join = None
        if self.join == "sum":
            lacking = [s for s in _SIDES if not hasattr(self.sides[s], "forward_inner")]
            if lacking:
                raise ValueError(f"side_by_side: the {' and '.join(lacking)} member cannot share a projection "
                                 "(no forward_inner); join 'sum' is built for members that can")
            # the members' columns of the shared buffer start at multiples of 8
            self.col = {"left": 0, "right": (self.left.inner_width + 7) // 8 * 8}
            self.join_width = self.col["right"] + (self.right.inner_width + 7) // 8 * 8

    def sub_mixers(self) -> List[Tuple[str, Mixer]]:
        return [(side, self.sides[side]) for side in _SIDES]

    def tensors(self) -> Dict[str, TensorDecl]:
        d: Dict[str, TensorDecl] = {}
        for side in _SIDES:
            for rel, decl in self.sides[side].tensors().items():
                d[f"{side}.{rel}"] = decl
            if self.join == "rms_mean":
                d[f"{side}.out"] = TensorDecl((self.hidden_size,), "norm")
        return d

    def load(self, fetch, dtype, device) -> None:
        for side in _SIDES:
            self.sides[side].load(lambda rel, _s=side: fetch(f"{_s}.{rel}"), dtype, device)
        if self.join == "sum":
            w = torch.zeros((self.hidden_size, self.join_width), dtype=dtype, device=device)
            for side in _SIDES:
                m = self.sides[side]
                w[:, self.col[side]:self.col[side] + m.inner_width] = m.inner_weight()
                m.w_o = w[:, self.col[side]:self.col[side] + m.inner_width]      # (one copy of the matrix is kept)
            self.w_join = w
            self.padded = self.join_width != self.left.inner_width + self.right.inner_width
            return
        self.w_left = fetch("left.out").to(torch.float32).to(device).contiguous()
        self.w_right = fetch("right.out").to(torch.float32).to(device).contiguous()

    def prepare(self, device, dtype) -> None:
        for side in _SIDES:
            self.sides[side].prepare(device, dtype)
            if self.join == "sum" and hasattr(self.sides[side], "set_out_scale"):
                self.sides[side].set_out_scale(self.scales[side])

    def kernel_libraries(self):
        libs = ["core"]
        for side in _SIDES:
            for name in self.sides[side].kernel_libraries():
                if name not in libs:
                    libs.append(name)
        return libs

    def weight_bytes(self) -> int:
        return sum(self.sides[s].weight_bytes() for s in _SIDES) + (8 * self.hidden_size if self.w_join is None else 0)

    def forward(self, x, step, cache):
        if self.join == "sum":
            make = torch.zeros if self.padded else torch.empty
            both = make((x.shape[0], self.join_width), dtype=x.dtype, device=x.device)
            for side in _SIDES:
                m = self.sides[side]
                m.forward_inner(x, step, cache[side], both[:, self.col[side]:self.col[side] + m.inner_width],
                                self.scales[side])
            return ops.linear(both, self.w_join, partial_ok=self.partial_ok)
        a = whole_output(self.left.forward(x, step, cache["left"]), x.dtype)
        b = whole_output(self.right.forward(x, step, cache["right"]), x.dtype)
        out = torch.empty((x.shape[0], self.hidden_size), dtype=x.dtype, device=x.device)
        ops.rms_pair_mean(out, a, getattr(self.left, "deferred_out_bias", None), self.w_left, b, self.w_right, self.eps)
        return out


register_part("mixer", "side_by_side", SideBySide)
