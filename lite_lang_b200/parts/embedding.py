"""Token embedding and the lm_head.

Embedding: ``litelang/models/qwen2/layer/pre_layer.py:15-19``.  Head:
``litelang/models/qwen2/layer/post_layer.py:20-22``; with tied embeddings it is
the embedding table itself (``layer_weights/post_layer_weights.py:10-15``), kept
as one buffer.  Logits are float32 on both paths.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Part, TensorDecl, register_part


class TokenEmbedding(Part):
    kind_family = "embedding"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        # ``scale``: a constant every row is multiplied by; ``residual``: "compute" (rows in the engine's
        # dtype) or "float32" (a model whose residual stream stays in 32-bit); ``tensor``: the table's
        # name under the prefix
        self.scale = float(spec.params.get("scale", 1.0))
        self.residual = str(spec.params.get("residual", "compute"))
        self.tensor = str(spec.params.get("tensor", "weight"))
        # ``streams``: a residual of several rows a token, [tokens, streams * hidden] float32, all starting as the row
        self.streams = int(spec.params.get("streams", 1))
        if self.streams != 1 and (self.residual != "float32" or self.scale != 1.0):
            raise ValueError("token_embedding: several streams are built for an unscaled float32 residual")
        if self.residual not in ("compute", "float32"):
            raise ValueError(f"token_embedding: residual {self.residual!r} is neither 'compute' nor 'float32'")
        if self.residual == "compute" and self.scale != 1.0:
            raise ValueError("token_embedding: a scale is built for a float32 residual stream only")
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor: TensorDecl((self.vocab_size, self.hidden_size))}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch(self.tensor).to(dtype).to(device).contiguous()

    def kernel_libraries(self):
        return ("core", "streams") if self.streams != 1 else ("core",)

    def forward(self, token_ids: torch.Tensor, num_tokens: int, status) -> torch.Tensor:
        if self.streams != 1:
            out = torch.empty((num_tokens, self.streams * self.hidden_size), dtype=torch.float32,
                              device=self.weight.device)
            ops.embed_streams(out, self.weight, token_ids[:num_tokens], self.streams, status)
            return out
        if self.residual == "float32":
            out = torch.empty((num_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
            ops.embed_scaled_f32(out, self.weight, token_ids[:num_tokens], self.scale, status)
            return out
        out = torch.empty((num_tokens, self.hidden_size), dtype=self.weight.dtype, device=self.weight.device)
        ops.embed_gather(out, self.weight, token_ids[:num_tokens], status)
        return out


class LMHead(Part):
    kind_family = "head"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.tied_to = spec.params.get("tied_to")
        self.tensor = str(spec.params.get("tensor", "weight"))
        # ``softcap`` c: logits <- c * tanh(logits / c)
        cap = spec.params.get("softcap")
        self.softcap = float(cap) if cap else None
        # ``scale``: a constant on the logits (applied to the float32 product)
        self.scale = float(spec.params.get("scale", 1.0))
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        # With tied embeddings a checkpoint may or may not repeat the table under lm_head.
        return {self.tensor: TensorDecl((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def load(self, fetch, dtype, device) -> None:
        if self.tied_to is None:
            self.weight = fetch(self.tensor).to(dtype).to(device).contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_logits(logits, self.scale)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
