"""Grouped-query attention over the paged cache with normalised operands and shaped scores.

One part, every mechanism a parameter, so that a design picks the ones it has:

``qkv_bias``          biases on q, k and v, added in the projection
``qk_norm``           None; "projection": q as one vector of all its heads (and k alike) through an RMS norm
                      with weights before the rotation; "head_unit": every q and k head divided by its root
                      mean square after the rotation
``value_norm``        every value head divided by its root mean square; the cache holds it so
``position``          a ``rope_computed`` part (partial rotation, interleaved or half-split pairs, scaled
                      frequencies with an amplitude on cos and sin)
``scale``             on q . k
``head_temperature``  a number a head on its scores
``head_mix``          the heads' scores mixed by a matrix [heads, heads] before the softmax: every head's score
                      of a (query, key) pair becomes a weighted sum of all heads' scores of that pair
``mask``, ``mask_size``  "causal"; "window": a token sees itself and the mask_size - 1 before it; "chunk": a
                      token sees the earlier tokens of its own chunk of mask_size positions, chunks counted
                      from the request's first token
``sink``              the softmax's denominator gains a 1: one more key of score 0 that carries no value;
                      "learned": the key's score is a number a head (tensor ``sink``), so the denominator gains
                      exp(sink_h); the score is not scaled, capped or biased
``head_gate``         every head's output times sigmoid(w_h . x), x being the input of the projections
``channel_gate``      every channel of every head's output times the sigmoid of its own gate input: the heads side
                      by side times sigmoid(W_g x) (tensor ``g`` [heads * vdim, hidden])
``distance_bias``     {"max": D}: a learned bias by distance, added to the scaled score: T[bucket(i - j), h] with
                      the table ``rel`` [B, heads] (B is the tensor's), bucket(n) = n below B // 2, then
                      B // 2 + floor(ln(n / (B // 2)) / ln(D / (B // 2)) * (B - B // 2)), capped at the last row
                      (which D has reached); {"buckets": B} only sizes random weights
``keep_first``        with a window: the request's first ``keep_first`` positions stay visible to every later
                      token (at their true distances); their pages stay with the request
``softcap``           the scaled score goes through cap * tanh(s / cap) (before any bias)
``query_temperature`` {"coef", "every"}: the query at position p is multiplied by
                      1 + coef * ln(floor((p + 1) / every) + 1)

The cache holds keys rotated and normalised and values normalised, one plane of pages; with a window or chunks
the pages that no later token can read go back to the pool while the request lives.  Scores, softmax weights,
norms and angles are float32 whatever the engine's dtype is.  q | k | v (| gate) are one product.

Kernels: in bfloat16 with head sizes 64 and 128, tensor cores (``attn_shaped``: prompt portions 128 rows a CTA,
single tokens with their keys split over CTAs; mixed heads as one wider query a head, made where q is
normalised; prompt portions of a design without mixed heads and sink: the plain attention's tcgen05 kernel, the
temperature on the queries and the gate in its epilogue); every other size, and float32, a block a token in
float32 arithmetic (``attention_modulated``).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, PagedKVNeed, TensorDecl, build_part, register_part

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
          "q_norm": "q.norm", "k_norm": "k.norm", "temperature": "temp", "mix": "talk", "gate": "g",
          "sink": "sink", "distance_bias": "rel"}


def distance_bucket(n: int, buckets: int, farthest: float) -> int:
    """The row of a distance-bias table for a key n positions back: one row a distance below buckets // 2, then
    rows in logarithmic steps, capped at the last row (which ``farthest`` has reached)."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(farthest / half) * (buckets - half))))


class ModulatedAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.vdim = int(p.get("value_head_dim") or self.head_dim)
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.eps = float(p.get("eps", 1e-6))
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.qk_norm = p.get("qk_norm")
        self.value_norm = bool(p.get("value_norm", False))
        self.head_temperature = bool(p.get("head_temperature", False))
        self.head_mix = bool(p.get("head_mix", False))
        self.sink = bool(p.get("sink", False))
        self.sink_learned = p.get("sink") == "learned"
        self.head_gate = bool(p.get("head_gate", False))
        self.channel_gate = bool(p.get("channel_gate", False))
        self.distance_bias = None if not p.get("distance_bias") else dict(p["distance_bias"])
        self.keep_first = int(p.get("keep_first") or 0)
        self.softcap = None if not p.get("softcap") else float(p["softcap"])
        qt = p.get("query_temperature")
        self.query_temperature = None if not qt else (float(qt["coef"]), int(qt["every"]))
        self.mask = str(p.get("mask", "causal"))
        size = p.get("mask_size")
        self.mask_size = None if size is None else int(size)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("modulated_attention: num_heads must be a multiple of num_kv_heads")
        if self.qk_norm not in ops.QK_NORM:
            raise ValueError(f"modulated_attention: qk_norm {self.qk_norm!r}; built: projection, head_unit, None")
        if self.mask not in ops.ATTN_MASK:
            raise ValueError(f"modulated_attention: mask {self.mask!r}; built: {', '.join(ops.ATTN_MASK)}")
        if self.mask != "causal" and (self.mask_size is None or self.mask_size <= 0):
            raise ValueError(f"modulated_attention: a {self.mask} mask needs a positive mask_size")
        if self.head_gate and self.channel_gate:
            raise ValueError("modulated_attention: a gate a head or a gate a channel, not both")
        if self.keep_first and self.mask != "window":
            raise ValueError("modulated_attention: keep_first goes with a window")
        if self.distance_bias is not None and not float(self.distance_bias.get("max", 0)) > 1:
            raise ValueError("modulated_attention: distance_bias needs 'max' (the distance of the last bucket) above 1")
        if self.query_temperature is not None and self.query_temperature[1] <= 0:
            raise ValueError("modulated_attention: query_temperature.every must be positive")
        if self.head_mix and (self.distance_bias is not None or self.softcap is not None or self.sink_learned):
            raise ValueError("modulated_attention: mixed heads with a distance bias, a cap or a learned sink are not built")
        pos = p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        if self.position is not None and not getattr(self.position, "computed", False):
            raise ValueError("modulated_attention: the position part must make its angles in the kernel "
                             "(rope_computed)")
        self.names = dict(_NAMES)
        self.names.update(dict(p.get("tensor_names") or {}))
        self.q_width = self.num_heads * self.head_dim
        self.k_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_kv_heads * self.vdim
        self.o_width = self.num_heads * self.vdim
        self.gate_offset = self.q_width + self.k_width + self.v_width
        self.w_in = self.b_in = self.w_o = None
        self.q_norm_w = self.k_norm_w = self.temperature = self.mix = None
        self.sink_w = self.bias_by_distance = None
        # mechanisms that the block-a-token kernel and the mma.sync kernel know and the tcgen05 kernel does not
        self.extended = bool(self.sink_learned or self.channel_gate or self.distance_bias is not None
                             or self.keep_first or self.softcap is not None or self.query_temperature is not None)

    def tensors(self) -> Dict[str, TensorDecl]:
        h, nm = self.hidden_size, self.names
        d = {nm["q"]: TensorDecl((self.q_width, h)), nm["k"]: TensorDecl((self.k_width, h)),
             nm["v"]: TensorDecl((self.v_width, h)), nm["o"]: TensorDecl((h, self.o_width))}
        if self.qkv_bias:
            d[nm["q_bias"]] = TensorDecl((self.q_width,), "bias")
            d[nm["k_bias"]] = TensorDecl((self.k_width,), "bias")
            d[nm["v_bias"]] = TensorDecl((self.v_width,), "bias")
        if self.qk_norm == "projection":
            d[nm["q_norm"]] = TensorDecl((self.q_width,), "norm")
            d[nm["k_norm"]] = TensorDecl((self.k_width,), "norm")
        if self.head_temperature:
            d[nm["temperature"]] = TensorDecl((self.num_heads,), "norm")
        if self.head_mix:
            d[nm["mix"]] = TensorDecl((self.num_heads, self.num_heads), "bias", std=0.2, eye=1.0)
        if self.head_gate:
            d[nm["gate"]] = TensorDecl((self.num_heads, h))
        if self.channel_gate:
            d[nm["gate"]] = TensorDecl((self.o_width, h))
        if self.sink_learned:
            d[nm["sink"]] = TensorDecl((self.num_heads,), "bias", std=1.0)
        if self.distance_bias is not None:
            # the number of buckets is the tensor's; random weights take ``buckets`` (32 if the design gives none)
            d[nm["distance_bias"]] = TensorDecl((None, self.num_heads), "bias", std=0.5,
                                                random_shape=(int(self.distance_bias.get("buckets") or 32),
                                                              self.num_heads))
        return d

    def load(self, fetch, dtype, device) -> None:
        nm = self.names
        gated = self.head_gate or self.channel_gate
        w = [fetch(nm[r]).to(dtype) for r in (("q", "k", "v", "gate") if gated else ("q", "k", "v"))]
        rows = sum(t.shape[0] for t in w)
        if rows % 8:      # rows of the product start on 16-byte boundaries (the tensor-core attention reads q so)
            w.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=dtype, device=w[0].device))
        self.w_in = torch.cat(w, dim=0).to(device).contiguous()
        if self.qkv_bias:
            b = [fetch(nm[r]).to(torch.float32) for r in ("q_bias", "k_bias", "v_bias")]
            self.b_in = torch.cat(b, dim=0).to(device).contiguous()
        self.w_o = fetch(nm["o"]).to(dtype).to(device).contiguous()

        def f32(name):
            return fetch(nm[name]).to(torch.float32).to(device).contiguous()

        if self.qk_norm == "projection":
            self.q_norm_w, self.k_norm_w = f32("q_norm"), f32("k_norm")
        if self.head_temperature:
            self.temperature = f32("temperature")
        if self.head_mix:
            self.mix = f32("mix")
        if self.sink_learned:
            self.sink_w = f32("sink")
        if self.distance_bias is not None:
            table = fetch(nm["distance_bias"]).to(torch.float32)
            if table.dim() != 2 or table.shape[0] < 2:
                raise ValueError(f"{self.prefix}{nm['distance_bias']}: a bias table needs at least two buckets")
            far = float(self.distance_bias["max"])
            if far <= table.shape[0] // 2:
                raise ValueError(f"{self.prefix}: distance_bias.max must lie beyond the table's exact buckets")
            # the bias a distance: from ceil(max) on every distance has the last bucket's
            rows = [distance_bucket(n, table.shape[0], far) for n in range(int(math.ceil(far)) + 1)]
            self.bias_by_distance = table[rows].to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.w_in.numel() * self.w_in.element_size() + self.w_o.numel() * self.w_o.element_size()

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim,
                           self.mask_size if self.mask == "window" else None,
                           None if self.vdim == self.head_dim else self.vdim,
                           self.mask_size if self.mask == "chunk" else None,
                           self.keep_first if self.mask == "window" else 0)

    def kernel_libraries(self):
        libs = ["core", "attn_mod"]
        if self.w_in is not None and self.w_in.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
            if self.head_dim in (64, 128) and self.vdim in (64, 128):
                libs.append("attn_shaped")
                if not self.head_mix and not self.sink and self.vdim == self.head_dim:
                    libs.append("attn_tc")
        return libs

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    # ------------------------------------------------------------------
    # A composite mixer that joins its members in one output projection asks for the heads side by side, times a
    # constant, written into its own buffer (``forward_inner``), and multiplies by ``inner_weight()`` itself.
    @property
    def inner_width(self) -> int:
        return self.o_width

    def inner_weight(self) -> torch.Tensor:
        return self.w_o

    def forward(self, x, step, cache):
        attn = torch.empty((x.shape[0], self.o_width), dtype=x.dtype, device=x.device)
        self.forward_inner(x, step, cache, attn)
        return ops.linear(attn, self.w_o, partial_ok=self.partial_ok)

    def forward_inner(self, x, step, cache, attn, out_scale: float = 1.0) -> None:
        n = x.shape[0]
        proj = ops.linear(x, self.w_in)                  # q | k | v (| gate inputs)
        pos = self.position
        # bfloat16 with head sizes the tensor-core kernel takes: mixed heads become one wider query a head
        shaped = ops.attn_shaped_supported(
            proj.dtype, self.num_kv_heads, self.head_dim, self.vdim, cache.page_size, proj.stride(0), self.head_mix)
        mixed_q = None
        if shaped and self.head_mix:
            mixed_q = torch.empty((n, self.num_heads * self.num_kv_heads * self.head_dim), dtype=proj.dtype,
                                  device=proj.device)
        # on that path a head's temperature goes onto its query before the query's one rounding
        fold = shaped and self.head_temperature and not self.head_mix
        ops.qkv_norm_rotate_store(
            proj, self.b_in, step.positions, None if pos is None else pos.freq,
            1.0 if pos is None else pos.amplitude, bool(pos is None or pos.interleaved), self.num_heads,
            self.num_kv_heads, self.head_dim, self.vdim, self.qk_norm, self.q_norm_w, self.k_norm_w, self.value_norm,
            self.eps, cache.slot_map if cache.writable else None, cache.k, cache.v, cache.page_size, step.status,
            head_mix=self.mix if mixed_q is not None else None,
            mix_temperature=self.temperature if (mixed_q is not None or fold) else None, mixed_q=mixed_q)
        if shaped:
            self.attend_shaped(attn, proj, mixed_q, step, cache, None if fold else self.temperature, out_scale)
        else:
            self.attend(attn, proj, step, cache, out_scale)

    def _gate(self, proj):
        if self.channel_gate:
            return proj[:, self.gate_offset:self.gate_offset + self.o_width]
        return proj[:, self.gate_offset:self.gate_offset + self.num_heads] if self.head_gate else None

    def attend(self, out, proj, step, cache, out_scale: float = 1.0) -> None:
        """Any sizes, both dtypes, float32 arithmetic: a block a token."""
        ops.attention_modulated(out, proj, proj.stride(0), self._gate(proj), cache.k, cache.v, cache.block_table,
                                step.token_req, step.req_slot, step.positions, proj.shape[0], self.num_heads,
                                self.num_kv_heads, self.head_dim, self.vdim, cache.page_size, self.mask,
                                self.mask_size, self.sink, self.scale, self.temperature, self.mix, step.status,
                                sink_values=self.sink_w, distance_bias=self.bias_by_distance,
                                keep_first=self.keep_first, softcap=self.softcap,
                                query_temperature=self.query_temperature, gate_channels=self.channel_gate,
                                out_scale=out_scale)

    def attend_shaped(self, out, proj, mixed_q, step, cache, temperature, out_scale: float = 1.0) -> None:
        """Tensor cores.  Single-token entries come first in a step: their keys are cut into parts of one or more
        stages of 64 keys, a CTA each (as many parts as the step's single tokens leave SMs for, so the order of a
        position's sums depends on how many tokens decode together, within rounding); the portions of prompts after
        them share the keys among 128 rows a CTA.  Portions whose scores are
        plain by now (no mixed heads, no sink, causal or a window, values as wide as keys; a temperature is on the
        queries already) go to the tcgen05 kernel of the plain attention, which takes the head gate."""
        q = proj if mixed_q is None else mixed_q
        group = self.num_heads // self.num_kv_heads
        n_single = step.num_single
        n_rest = step.num_entries - n_single
        tail = (self.num_heads, self.num_kv_heads, self.head_dim, self.vdim, cache.page_size, self.mask,
                self.mask_size, self.sink, self.scale, step.status)
        head = (out, q, q.stride(0), mixed_q is not None, self._gate(proj), temperature, cache.k, cache.v,
                cache.block_table)
        more = dict(sink_values=self.sink_w, distance_bias=self.bias_by_distance, keep_first=self.keep_first,
                    softcap=self.softcap, query_temperature=self.query_temperature, gate_channels=self.channel_gate,
                    out_scale=out_scale)
        if n_single > 0:
            if self.mask == "causal":
                stages = (int(step.max_kv_len) + 63) // 64 + 1
            else:
                stages = (self.mask_size + 62) // 64 + 1
            # as many parts as give every SM a CTA, at most one part a stage and 32 parts: 8 tokens on 2 kv heads
            # with a window of 512 get 9 parts of one stage; 64 tokens one part each (and no join)
            ctas = n_single * self.num_kv_heads * ((group + 127) // 128)
            # (without a window or chunks a token's walk is as long as its context: two CTAs an SM then)
            slots = ops.sm_count(out.device) * (2 if self.mask == "causal" else 1)
            want = max(1, min(32, slots // ctas))
            span = (stages + want - 1) // want
            nsplit = (stages + span - 1) // span
            ops.attn_shaped(*head, step.cu_q, step.ctx_len, step.req_slot, n_single, n_single * ((group + 127) // 128),
                            *tail, nsplit=nsplit, span=span, **more)
        if (n_rest > 0 and mixed_q is None and temperature is None and not self.sink and self.vdim == self.head_dim
                and not self.extended and out_scale == 1.0
                and self.mask in ("causal", "window") and ops.TC_ENABLED
                and ops.attn_prefill_tc_supported(proj.dtype, self.head_dim, cache.page_size, proj.stride(0), group)):
            window = self.mask_size if self.mask == "window" else None
            key = ("attn_prefill_tc", group, window)
            plan = step.scratch.get(key)
            if plan is None:
                rest_entries = step.entries[n_single:]
                ctxs = getattr(step, "entry_ctx", None)
                if ctxs is not None:
                    plan = ops.attn_prefill_tc_plan(
                        [(ctxs[n_single + i], len(e.tokens)) for i, e in enumerate(rest_entries)], group, window,
                        self.num_kv_heads, 2 * ops.sm_count(proj.device))
                else:
                    blocks = ops.attn_prefill_tc_blocks((len(e.tokens) for e in rest_entries), group)
                    plan = (blocks, ops.attn_prefill_tc_splits(blocks, self.num_kv_heads, proj.device), 8)
                step.scratch[key] = plan
            ops.attn_prefill_tc(out, proj, proj.stride(0), cache.k, cache.v, cache.block_table, step.cu_q[n_single:],
                                step.ctx_len[n_single:], step.req_slot[n_single:], n_rest, plan[0], self.num_heads,
                                self.num_kv_heads, self.head_dim, cache.page_size, window, self.scale, step.status,
                                nsplit=plan[1], split_len=plan[2], gate=self._gate(proj))
        elif n_rest > 0:
            key = ("attn_shaped", group)
            blocks = step.scratch.get(key)
            if blocks is None:
                blocks = step.scratch[key] = ops.attn_shaped_blocks(
                    (len(e.tokens) for e in step.entries[n_single:]), group)
            ops.attn_shaped(*head, step.cu_q[n_single:], step.ctx_len[n_single:], step.req_slot[n_single:], n_rest,
                            blocks, *tail, **more)


register_part("mixer", "modulated_attention", ModulatedAttention)
