"""Routed feed-forward (mixture of experts), optionally with an expert that every token uses.

A router scores all ``experts`` in float32 (scores = ``score``(W_router x): "softmax" over all experts, or
"sigmoid"), the ``top`` largest are chosen, and the output is the sum of the chosen experts' outputs weighted
by their scores (divided by their sum first if ``renormalize``).  An expert is down(act(up x)) without biases,
act = ``activation`` ("relu2": the square of relu; "silu"; "gelu_tanh"; "gelu": the erf form).  ``shared_ff`` > 0 adds an expert of
that width (tensors ``shared.up``, ``shared.down``) that runs for every token with weight 1.

Two ways through the experts, both without the host ever knowing who chose whom:

* few tokens (decode steps, short portions) and the float32 path: all experts' up matrices are stacked into one
  (the shared expert's rows first), so the first product is one product over all hidden units; the activation
  kernel multiplies each unit by its expert's weight for the token (an exact zero for experts that were not
  chosen), and one product with the stacked down matrices gives the weighted sum.  With few tokens a step reads
  every expert's weights anyway, and that is what bounds it.
* many tokens (``GROUPED_MIN_TOKENS``; bfloat16; widths that are multiples of 8): the (token, expert) pairs are
  put in the order of the experts on the device, the chosen tokens' rows gathered, and two grouped library
  products (a group an expert, the groups' ends a device array) do only the chosen experts' arithmetic; the
  pairs' results are added per token in the order of the pairs, onto the shared expert's output.

A token's result does not depend on which other tokens are in the step (beyond which of the two ways it takes).

Further parameters, for designs that differ:
``gated``         experts have a gate: down(a * sigmoid(``swish_alpha`` a) * (c + 1)) with a = min(gate x, ``limit``)
                  and c = clamp(up x, -limit, limit) (tensors ``e<i>.gate`` beside ``up`` and ``down``); the shared
                  expert has the same form with ``shared_limit``.
``score``         "softmax_top": the ``top`` largest logits are chosen, weighted by the softmax over the chosen only.
``router_bias``   a bias on the router's logits (tensor ``router.b``).
``shared_gate``   the shared expert's output is multiplied by sigmoid(w . x), one number a token (``shared.sg``).
``weight_on``     "output" (the sum of w_e expert_e(x)) or "input": the sum of expert_e(w_e x), the weight
                  multiplying what the expert reads.  Since U (w x) = w (U x) the first product is the same and
                  the weight goes inside the activation: down(act(w (up x))).
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_part


class RoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.E = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_ff"])
        self.shared_ff = int(p.get("shared_ff") or 0)
        self.activation = str(p.get("activation", "relu2"))
        self.score = str(p.get("score", "softmax"))
        self.renormalize = bool(p.get("renormalize", False))
        self.gated = bool(p.get("gated", False))
        self.limit = float(p.get("limit") or 0.0)
        self.shared_limit = float(p.get("shared_limit") or self.limit)
        self.swish_alpha = float(p.get("swish_alpha", 1.702))
        self.router_bias = bool(p.get("router_bias", False))
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_ff > 0
        self.weight_on = str(p.get("weight_on", "output"))
        if self.weight_on not in ("output", "input") or (self.gated and self.weight_on == "input"):
            raise ValueError("routed_experts: weight_on is 'output' or (experts without a gate) 'input'")
        self.weight_in = self.weight_on == "input"
        if self.gated and not (self.limit > 0 and self.shared_limit > 0):
            raise ValueError("routed_experts: gated experts take a positive limit")
        if (not self.gated and self.activation not in ops.MOE_ACT) or self.score not in ops.MOE_SCORE:
            raise ValueError(f"routed_experts: activation {self.activation!r} / score {self.score!r} is not built")
        if not (0 < self.top <= self.E <= 256):
            raise ValueError("routed_experts: 0 < top <= experts <= 256")
        self.w_up = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        d = {"router": TensorDecl((self.E, h), std=0.3)}
        if self.router_bias:
            d["router.b"] = TensorDecl((self.E,), "bias", std=0.3)
        names = [f"e{e}" for e in range(self.E)] + (["shared"] if self.shared_ff else [])
        for nm in names:
            ff = self.shared_ff if nm == "shared" else self.ff
            if self.gated:
                d[f"{nm}.gate"] = TensorDecl((ff, h))
            d[f"{nm}.up"] = TensorDecl((ff, h))
            d[f"{nm}.down"] = TensorDecl((h, ff))
        if self.shared_gate:
            d["shared.sg"] = TensorDecl((1, h), std=0.3)
        return d

    def load(self, fetch, dtype, device) -> None:
        # the first product's rows: the shared expert's, then expert by expert; with a gate, an expert's gate
        # rows come before its up rows
        names = (["shared"] if self.shared_ff else []) + [f"e{e}" for e in range(self.E)]
        ups = []
        for nm in names:
            if self.gated:
                ups.append(fetch(f"{nm}.gate"))
            ups.append(fetch(f"{nm}.up"))
        downs = [fetch(f"{nm}.down") for nm in names]
        self.w_up = torch.cat([u.to(dtype) for u in ups], dim=0).to(device).contiguous()
        self.w_down = torch.cat([w.to(dtype) for w in downs], dim=1).to(device).contiguous()
        router = [fetch("router").to(torch.float32)]
        if self.shared_gate:
            router.append(fetch("shared.sg").to(torch.float32).reshape(1, -1))   # one more row: the shared expert's gate
        self.w_router = torch.cat(router, dim=0).to(device).contiguous()
        self.b_router = fetch("router.b").to(torch.float32).to(device).contiguous() if self.router_bias else None
        # views for the grouped way: the experts' up matrices [E, ff, hidden] inside the stacked one; their down
        # matrices [E, hidden, ff] as strided views of the stacked one's columns
        sff, ff, E, h = self.shared_ff, self.ff, self.E, self.hidden_size
        if self.gated:
            sff, ff = 2 * sff, 2 * ff
        self.w_up_experts = self.w_up[sff:].view(E, ff, h)
        sff, ff = self.shared_ff, self.ff
        self.w_down_experts = self.w_down[:, sff:].unflatten(1, (E, ff)).permute(1, 0, 2)
        self.grouped = (dtype == torch.bfloat16 and h % 8 == 0 and ff % 8 == 0 and sff % 8 == 0
                        and ops.grouped_product_available())

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down, self.w_router))

    _shared_w = None

    def kernel_libraries(self):
        libs = ["core", "moe"]
        if self.w_up is not None and self.w_up.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    def route(self, x):
        n, dev = x.shape[0], x.device
        gates = torch.empty((n, self.E), dtype=torch.float32, device=dev)
        top_idx = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        top_w = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        self._shared_w = torch.empty((n,), dtype=torch.float32, device=dev) if self.shared_gate else None
        ops.moe_router(x, self.w_router, gates, top_idx, top_w, self.top, self.score, self.renormalize,
                       bias=self.b_router, shared_w=self._shared_w)
        return gates, top_idx, top_w

    GROUPED_MIN_TOKENS = 128

    def forward(self, x, step):
        gates, idx, wts = self.route(x)
        if self.grouped and x.shape[0] >= self.GROUPED_MIN_TOKENS and not getattr(step, "captured", False):
            try:
                return self._forward_grouped(x, idx, wts)
            except (RuntimeError, NotImplementedError) as exc:      # a shape the library's grouped product refuses
                import sys
                print(f"[lite_lang_b200] routed_experts {self.prefix}: grouped product refused ({str(exc)[:120]}); "
                      "the stacked way is used instead", file=sys.stderr)
                self.grouped = False
        hidden = ops.linear(x, self.w_up)
        if self.gated:
            hidden = ops.moe_gated_act(hidden, gates, self._shared_w, self.shared_ff, self.ff, self.E, self.limit,
                                       self.shared_limit, self.swish_alpha)
        else:
            ops.moe_act(hidden, gates, self.shared_ff, self.ff, self.E, self.activation, self.weight_in)
        # (few tokens and many hidden units: float32 partial sums of a split inner dimension, added up by the norm)
        return ops.linear(hidden, self.w_down, partial_ok=True)


    def _forward_grouped(self, x, idx, wts):
        sff = self.shared_ff
        base = None
        if sff and self.gated:
            hs = ops.linear(x, self.w_up[:2 * sff])
            hs = ops.moe_row_gated_act(hs, self._shared_w, self.shared_limit, self.swish_alpha)
            base = ops.linear(hs, self.w_down[:, :sff])
        elif sff:
            hs = ops.linear(x, self.w_up[:sff])
            ops.moe_act(hs, wts, sff, self.ff, 0, self.activation)      # (no routed columns: every weight is 1)
            base = ops.linear(hs, self.w_down[:, :sff])
        ends, row_token, row_w, pair_row = ops.moe_sort(idx, wts, self.E)
        rows = ops.moe_gather_rows(x, row_token)
        hidden = ops.grouped_product(rows, self.w_up_experts, ends)
        if self.gated:
            hidden = ops.moe_row_gated_act(hidden, row_w, self.limit, self.swish_alpha)
        else:
            ops.moe_row_act(hidden, row_w, self.activation, self.weight_in)
        y = ops.grouped_product(hidden, self.w_down_experts, ends)
        return ops.moe_combine(base, y, pair_row)


register_part("feed_forward", "routed_experts", RoutedExperts)
