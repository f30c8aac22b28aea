"""State-space mixer with a scalar decay a head and token (Mamba-2, "state-space duality"): a recurrent mixer
with a matrix state a head.

One product gives [z | x | B | C | dt]: with inner = ``heads`` x ``head_dim``, z and x are inner wide, B and C
``groups`` x ``state`` wide, dt ``heads`` wide.  x, B and C together pass a causal convolution a channel
(``conv_taps`` weights, the last for the token itself, and a bias; zeros before the request's start) and SiLU.
dt = softplus(dt + dt_bias), without a clamp.  Per head h, which reads the B and C of group h // (heads / groups):

    S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T,      y_t = S_t^T C_t + D_h x_t      (S is state x head_dim)

The heads' y side by side are multiplied by silu(z), then every one of ``norm_groups`` equal parts is divided by
its root mean square (eps inside the root), times the weight ``norm``; then W_o.

A request's state is all zeros before its first token; it is float32 and lives, with the convolution's last
``conv_taps`` - 1 inputs behind it, in the request's record of the cache manager's state pool, so a request goes
on in a later step, alone or beside others, from where it stopped.  Everything between the convolution and the
output projection is float32: step sizes, decays, the state, the scan's operands, gate and norm.
Tensors: ``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, StateNeed, TensorDecl, register_part


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class StateSpaceDuality(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["heads"])
        self.P = int(p["head_dim"])
        self.N = int(p["state"])
        self.G = int(p.get("groups", 1))
        self.taps = int(p.get("conv_taps", 4))
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.H * self.P
        self.C = self.inner + 2 * self.G * self.N          # channels of the convolution: x | B | C
        if self.G <= 0 or self.H % self.G:
            raise ValueError("state_space_duality: heads must be a multiple of groups")
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError("state_space_duality: heads * head_dim must be a multiple of norm_groups")
        if self.taps < 1 or not (0 < self.N <= 256):
            raise ValueError("state_space_duality: conv_taps >= 1 and a state of 1 to 256 numbers are built")
        self.state_floats = self.H * self.P * self.N
        self.w_in = None
        self._scaled_norm = (1.0, None)

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        return {
            "in": TensorDecl((2 * self.inner + 2 * self.G * self.N + self.H, h)),
            "conv": TensorDecl((self.C, self.taps), "bias", std=0.4),
            "conv.b": TensorDecl((self.C,), "bias"),
            "dt_bias": TensorDecl((self.H,), "bias", std=0.5),
            "A_log": TensorDecl((self.H,), "bias", std=0.5, mean=-1.0),
            "D": TensorDecl((self.H,), "bias", std=0.5, mean=1.0),
            "norm": TensorDecl((self.inner,), "norm"),
            "o": TensorDecl((h, self.inner)),
        }

    def load(self, fetch, dtype, device) -> None:
        def f32(name):
            return fetch(name).to(torch.float32).to(device).contiguous()

        # the product's rows: z, then x | B | C, then dt; every segment starts at a multiple of 8 rows
        w = fetch("in").to(dtype)
        segs = (("z", w[:self.inner]), ("x", w[self.inner:self.inner + self.C]), ("dt", w[self.inner + self.C:]))
        self.off, rows, at = {}, [], 0
        for name, part in segs:
            self.off[name] = at
            rows.append(part)
            pad = _pad8(part.shape[0]) - part.shape[0]
            if pad:
                rows.append(torch.zeros((pad, self.hidden_size), dtype=dtype, device=part.device))
            at += _pad8(part.shape[0])
        self.w_in = torch.cat(rows, dim=0).to(device).contiguous()
        self.conv_w, self.conv_b = f32("conv"), f32("conv.b")
        self.dt_bias, self.A_log, self.D, self.norm_w = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")
        self.w_o = fetch("o").to(dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.conv_w, self.norm_w))

    def cache_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * self.C,), "float32")

    def kernel_libraries(self):
        libs = ["core", "ssd", "linear_attn"]
        if self.w_in is not None and self.w_in.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    # (see ``ModulatedAttention.forward_inner``: for a composite mixer that joins its members in one projection)
    @property
    def inner_width(self) -> int:
        return self.inner

    def inner_weight(self) -> torch.Tensor:
        return self.w_o

    def set_out_scale(self, out_scale: float) -> None:
        """A constant on the output rides on the norm's weight (float32); made once, before any captured step."""
        if out_scale != 1.0 and self._scaled_norm[0] != out_scale:
            self._scaled_norm = (out_scale, (self.norm_w * out_scale).contiguous())

    def forward(self, x, step, cache):
        out = torch.empty((x.shape[0], self.inner), dtype=x.dtype, device=x.device)
        self.forward_inner(x, step, cache, out)
        return ops.linear(out, self.w_o, partial_ok=self.partial_ok)

    def forward_inner(self, x, step, cache, out, out_scale: float = 1.0) -> None:
        n, dev = x.shape[0], x.device
        proj = ops.linear(x, self.w_in)
        f32 = dict(dtype=torch.float32, device=dev)
        xbc = torch.empty((n, self.C), **f32)
        dt = torch.empty((n, self.H), **f32)
        decay = torch.empty((n, self.H), **f32)
        ops.ssd_prepare(proj, self.off["x"], self.off["dt"], self.conv_w, self.conv_b, self.A_log, self.dt_bias,
                        cache.state, self.state_floats, step, xbc, dt, decay, cache.writable)
        y = torch.empty((n, self.inner), **f32)
        # the scan of the decayed linear attention: q = C, k = B (a group's, shared by its heads), v = x
        ops.decay_scan(xbc, self.inner + self.G * self.N, self.inner, 0, None, cache.state, step, y, self.H, self.N,
                       self.P, cache.writable, heads_per_group=self.H // self.G, token_decay=decay, token_scale=dt,
                       skip=self.D)
        self.set_out_scale(out_scale)
        ops.ssd_gated_norm(out, y, proj[:, self.off["z"]:self.off["z"] + self.inner],
                           self.norm_w if out_scale == 1.0 else self._scaled_norm[1], self.eps, self.norm_groups)


register_part("mixer", "state_space_duality", StateSpaceDuality)
