"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * w, computed in float32.

Formula: ``litelang/kernel/develop_rmsnorm/rms_norm.py:11-17,43-53``; used before
the mixer, before the feed-forward and before the lm_head
(``litelang/models/qwen2/layer/transformer_layer.py:86-92``, ``post_layer.py:43-45``).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Norm, ResidualCopy, StreamWrite, TensorDecl, register_part, whole_output


class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch("weight").to(torch.float32).to(device).contiguous()

    def split_params(self):
        return self.weight, self.eps

    def forward(self, x, out=None):
        if out is None:
            out = torch.empty_like(x)
        ops.rmsnorm(out, x, self.weight, self.eps)
        return out

    def add_forward(self, residual, delta, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, residual.shape[1]), dtype=residual.dtype, device=residual.device)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, rows)
        return out


class LayerNormF32Residual(Norm):
    """Layer norm with a weight and no bias, y = (x - mean) / sqrt(var + eps) * w, over a residual stream
    that is kept in float32 whatever the engine's dtype is; its output has the engine's dtype.

    ``add_forward`` takes the not yet added outputs of the parts before it as one tensor or as a tuple of
    up to two (a block whose mixer and feed-forward read the same norm hands on both): they are added to
    each other, then to the residual, in float32.  ``tensor`` is the weight's name under the prefix.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor: TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch(self.tensor).to(torch.float32).to(device).contiguous()
        self.out_dtype = dtype

    def forward(self, x, out=None):
        return self.add_forward(x, None)

    def add_forward(self, residual, delta, rows=None):
        if residual.dtype != torch.float32:
            raise TypeError("layer_norm_f32: the residual stream of this norm is float32")
        if isinstance(delta, ResidualCopy):      # nothing is pending
            delta = None
        deltas = [d for d in (delta if isinstance(delta, (tuple, list)) else (delta,)) if d is not None]
        if len(deltas) > 2:
            raise ValueError("layer_norm_f32: at most two pending outputs can be added in the norm")
        # one of them may come as float32 partial sums of a product split over its inner dimension
        partial = next((d for d in deltas if d.dim() == 3), None)
        deltas = [whole_output(d, self.out_dtype) for d in deltas if d is not partial] + [None, None]
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, residual.shape[1]), dtype=self.out_dtype, device=residual.device)
        ops.add_layernorm(out, residual, deltas[0], deltas[1], self.weight, self.eps, rows, partial)
        return out


class DynamicTanh(Norm):
    """Dynamic tanh: y = tanh(alpha * u) * w + b with a scalar alpha; no mean, no variance.

    It reads a float32 residual of ``streams`` rows a token, laid out [tokens, streams * hidden]:
    u = sum_s read[s] X[s] (``read`` None: the plain sum).  ``add_forward`` first applies a pending
    ``StreamWrite`` (X[t] <- sum_s mix[s, t] X[s] + write[t] y), all in the same pass; with one stream a plain
    pending output is the residual sum X <- X + y.  The output has the engine's dtype.  Tensors: ``tensor``
    (w), ``tensor`` + ".b", ``tensor`` + ".alpha" under the prefix.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.streams = int(spec.params.get("streams", 1))
        self.tensor = str(spec.params.get("tensor", "weight"))
        if not (1 <= self.streams <= 8):
            raise ValueError("dynamic_tanh: 1 to 8 streams are built")
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None
        self._ones = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor: TensorDecl((self.hidden_size,), "norm"),
                self.tensor + ".b": TensorDecl((self.hidden_size,), "bias"),
                self.tensor + ".alpha": TensorDecl((), "bias", std=0.1, mean=0.6)}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch(self.tensor).to(torch.float32).to(device).contiguous()
        self.bias = fetch(self.tensor + ".b").to(torch.float32).to(device).contiguous()
        self.alpha = fetch(self.tensor + ".alpha").to(torch.float32).reshape(1).to(device).contiguous()
        self.out_dtype = dtype
        self._ones = torch.ones(1, dtype=torch.float32, device=device)

    def kernel_libraries(self):
        return ("core", "streams")

    def weight_bytes(self) -> int:
        return 4 * (2 * self.hidden_size + 1)

    def forward(self, x, out=None):
        return self.add_forward(x, None)

    def add_forward(self, residual, delta, rows=None, read=None):
        if residual.dtype != torch.float32 or residual.shape[1] != self.streams * self.hidden_size:
            raise TypeError("dynamic_tanh: the residual is float32 [tokens, streams * hidden]")
        y = mix = write = None
        if isinstance(delta, StreamWrite):
            y, mix, write = delta
        elif delta is not None:
            if self.streams != 1:
                raise TypeError("dynamic_tanh: a residual of several streams takes a StreamWrite")
            y, mix, write = delta, self._ones, self._ones
        if y is not None and y.dim() == 2 and y.dtype != self.out_dtype:
            y = y.to(self.out_dtype)
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.hidden_size), dtype=self.out_dtype, device=residual.device)
        ops.stream_tanh_norm(out, residual, self.streams, self.alpha, self.weight, self.bias, read, y, mix, write, rows)
        return out


class OutputLayerNorm(Norm):
    """Layer norm with a weight and no bias on a sublayer's *output*, which is then added to a float32 residual
    stream: residual += (y - mean) / sqrt(var + eps) * w.  The sublayers of such a layer read the residual
    itself, so the pass that writes the residual also leaves it rounded to the engine's dtype for the products
    that read it next (``add_into`` returns that copy; on the float32 path it is the residual).

    ``y`` may be float32 partial sums [parts, tokens, hidden] of a product split over its inner dimension;
    they are added up in float32 and not rounded.  ``tensor`` is the weight's name under the prefix.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor: TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch(self.tensor).to(torch.float32).to(device).contiguous()
        self.out_dtype = dtype

    def add_into(self, residual: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if residual.dtype != torch.float32:
            raise TypeError("layer_norm_out: the residual stream of this norm is float32")
        if y.dim() == 2 and y.dtype != self.out_dtype:
            y = y.to(self.out_dtype)
        copy = None
        if self.out_dtype != torch.float32:
            copy = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        ops.layernorm_into_residual(residual, y.contiguous(), self.weight, self.eps, copy)
        return residual if copy is None else copy

    def forward(self, x, out=None):
        raise TypeError("layer_norm_out norms a sublayer's output into the residual stream: use add_into")


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm_out", OutputLayerNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
register_part("norm", "layer_norm_f32", LayerNormF32Residual)
