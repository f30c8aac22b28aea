"""SiLU-gated feed-forward: down(silu(gate(x)) * up(x)), no biases.

``litelang/models/qwen2/layer/transformer_layer.py:79-83``; gate and up are fused
into one projection whose first I columns are the gate
(``litelang/models/qwen2/layer_weights/load_weights.py:160-172``).  The
activation is evaluated in float32 (``litelang/kernel/develop_silu_and_mul/
silu_and_mul.py:43-50`` rounds the gate's SiLU first; here the whole expression is
rounded once).
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, NormSplit, TensorDecl, register_part


class GatedMLP(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.intermediate_size = int(spec.params["intermediate_size"])
        act = spec.params.get("activation", "silu")
        if act not in ops.GATE_ACT:
            raise ValueError(f"gated_mlp: activation {act!r} is not built ({', '.join(ops.GATE_ACT)})")
        self.activation = act
        # ``tensor_names``: (gate, up, down) under the prefix, for checkpoints that call them otherwise
        self.names = tuple(spec.params.get("tensor_names") or ("gate_proj.weight", "up_proj.weight",
                                                               "down_proj.weight"))
        self.w_gate_up = None
        self.w_down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names[0]: TensorDecl((i, h)),
            self.names[1]: TensorDecl((i, h)),
            self.names[2]: TensorDecl((h, i)),
        }

    def load(self, fetch, dtype, device) -> None:
        gate = fetch(self.names[0]).to(dtype)
        up = fetch(self.names[1]).to(dtype)
        self.w_gate_up = torch.cat((gate, up), dim=0).to(device).contiguous()
        self.w_down = fetch(self.names[2]).to(dtype).to(device).contiguous()

    def kernel_libraries(self):
        bf16 = self.w_down is not None and self.w_down.dtype == torch.bfloat16
        return ["core", "gemm_smallm", "gemm_stream", "gemm_tc", "gemm_pair"] if bf16 else ["core"]

    def weight_bytes(self) -> int:
        return self.w_gate_up.numel() * self.w_gate_up.element_size() + self.w_down.numel() * self.w_down.element_size()

    accumulates = True
    takes_norm_split = True

    def accepts_norm_split(self, rows) -> bool:
        return self.activation == "silu" and ops.gated_scaled_supported(rows, self.w_gate_up)

    def forward(self, x, step, residual=None):
        if isinstance(x, NormSplit):    # the norm before this part, left to its first product
            act = ops.gemm_stream_gated_scaled(x.scaled, self.w_gate_up, x.sumsq, x.eps, step.status)
        else:
            act = ops.gated_linear(x, self.w_gate_up, self.activation)
        if residual is not None and ops.accumulate_preferred(act, self.w_down):
            ops.linear_accumulate(act, self.w_down, residual)
            return None
        return ops.linear(act, self.w_down, partial_ok=True)


class DenseMLP(FeedForward):
    """Feed-forward without a gate: down(act(up(x))), no biases; ``activation`` gelu_tanh (the tanh form of
    GELU), relu, silu or relu2 (the square of relu), evaluated in float32.  ``tensor_names``: (up, down) under the prefix."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.intermediate_size = int(spec.params["intermediate_size"])
        act = spec.params.get("activation", "gelu_tanh")
        if act not in ops.ROW_ACT:
            raise ValueError(f"dense_mlp: activation {act!r} is not built ({', '.join(ops.ROW_ACT)})")
        self.activation = act
        self.names = tuple(spec.params.get("tensor_names") or ("up_proj.weight", "down_proj.weight"))
        self.w_up = None
        self.w_down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {self.names[0]: TensorDecl((i, h)), self.names[1]: TensorDecl((h, i))}

    def load(self, fetch, dtype, device) -> None:
        self.w_up = fetch(self.names[0]).to(dtype).to(device).contiguous()
        self.w_down = fetch(self.names[1]).to(dtype).to(device).contiguous()

    def kernel_libraries(self):
        bf16 = self.w_down is not None and self.w_down.dtype == torch.bfloat16
        return ["core", "gemm_smallm", "gemm_stream", "gemm_tc", "gemm_pair"] if bf16 else ["core"]

    def weight_bytes(self) -> int:
        return self.w_up.numel() * self.w_up.element_size() + self.w_down.numel() * self.w_down.element_size()

    def forward(self, x, step):
        act = ops.linear_act(x, self.w_up, self.activation)
        return ops.linear(act, self.w_down, partial_ok=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "dense_mlp", DenseMLP)
