"""Latent attention: keys and values expanded from one cached latent vector per token, sliding window.

Per token the input is projected to ``heads`` queries, each [``dim`` plain | ``rot_dim`` rotated], and to
``kv_rank + rot_dim`` numbers: the first ``kv_rank``, RMS-normed with a weight, are the latent c; the last
``rot_dim`` are one rotated key part shared by all heads.  A head's plain key is Uk_h c, its value Uv_h c;
score = (q_plain . k_plain + q_rot . k_rot) * ``scale``; position i sees j with 0 <= i - j < ``window``
(None: every earlier position); softmax; output projection over the concatenated heads.

Only c and the rotated key part are cached: ``kv_rank + rot_dim`` numbers a token in one plane of a paged
group with one kv head and no value plane.  Nothing per head is expanded from the cache either: since
q_plain . (Uk_h c) = (Uk_h^T q_plain) . c, the queries are taken into the latent space by a batched product
over heads, attention runs there (keys: the cached rows; values: their first ``kv_rank`` numbers), and a
second batched product expands each head's weighted sum of latents with Uv_h.

Rotation: interleaved pairs (2i, 2i+1) of the rotated part's first ``rot_dims`` numbers turn by
position * ``rot_base``^(-2i / rot_dims); the rest passes unchanged.  Angles (float32 position times a
float32 frequency rounded from float64), the latent's norm, scores and softmax are float32.

Further parameters, for designs that differ:
``q_rank``       the queries go through a latent of their own: c_q = RMS norm (weight ``dq.norm``) of W_dq x
                 (``q_rank`` numbers), q = W_uq c_q (tensors ``dq``, ``dq.norm``, ``uq`` in the place of ``q``)
``sink``         every head's softmax has one more key, of the learned score ``sink`` [heads], without a value
``rot_scaling``  (``factor``, ``original``, ``fast``, ``slow``) the slow frequencies stretched and an amplitude on
                 cos and sin, as ``rope_computed`` makes them
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import PartSpec
from ..config.spec import PartSpec as _PartSpec
from .base import Mixer, PagedKVNeed, TensorDecl, build_part, register_part


class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["heads"])
        self.d = int(p["dim"])
        self.r = int(p["rot_dim"])
        self.dv = int(p["vdim"])
        self.R = int(p["kv_rank"])
        self.window = None if p.get("window") is None else int(p["window"])
        self.scale = float(p.get("scale", (self.d + self.r) ** -0.5))
        self.rot_base = float(p.get("rot_base", 10000.0))
        self.rot_dims = int(p.get("rot_dims", self.r))
        self.eps = float(p["eps"])
        self.q_rank = None if p.get("q_rank") is None else int(p["q_rank"])
        self.sink = bool(p.get("sink", False))
        self.rot_scaling = None if not p.get("rot_scaling") else dict(p["rot_scaling"])
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.r):
            raise ValueError("latent_attention: rot_dims must be even and at most rot_dim")
        if self.R > 512:
            raise ValueError("latent_attention: a latent of more than 512 numbers is not built")
        if self.window is not None and self.window <= 0:
            raise ValueError("latent_attention: the window must be positive")
        self.w_in = None
        self.w_uq = self.q_norm_w = self.sink_w = None
        self.amplitude = 1.0

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        d: Dict[str, TensorDecl] = {}
        if self.q_rank is None:
            d["q"] = TensorDecl((self.H * (self.d + self.r), h))
        else:
            d["dq"] = TensorDecl((self.q_rank, h))
            d["dq.norm"] = TensorDecl((self.q_rank,), "norm")
            d["uq"] = TensorDecl((self.H * (self.d + self.r), self.q_rank))
        if self.sink:
            d["sink"] = TensorDecl((self.H,), "bias", std=1.0)
        d.update(self._kv_tensors())
        return d

    def _kv_tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        return {
            "dkv": TensorDecl((self.R + self.r, h)),
            "dkv.norm": TensorDecl((self.R,), "norm"),
            "uk": TensorDecl((self.H * self.d, self.R)),
            "uv": TensorDecl((self.H * self.dv, self.R)),
            "o": TensorDecl((h, self.H * self.dv)),
        }

    def load(self, fetch, dtype, device) -> None:
        q = fetch("q" if self.q_rank is None else "dq").to(dtype)
        if self.q_rank is not None:
            self.w_uq = fetch("uq").to(dtype).to(device).contiguous()
            self.q_norm_w = fetch("dq.norm").to(torch.float32).to(device).contiguous()
        if self.sink:
            self.sink_w = fetch("sink").to(torch.float32).to(device).contiguous()
        self.kv_off = (q.shape[0] + 7) // 8 * 8
        rows = [q]
        if self.kv_off != q.shape[0]:
            rows.append(torch.zeros((self.kv_off - q.shape[0], self.hidden_size), dtype=dtype, device=q.device))
        rows.append(fetch("dkv").to(dtype))
        self.w_in = torch.cat(rows, dim=0).to(device).contiguous()
        self.norm_w = fetch("dkv.norm").to(torch.float32).to(device).contiguous()
        self.w_uk = fetch("uk").to(dtype).to(device).contiguous().view(self.H, self.d, self.R)
        self.w_uv_t = fetch("uv").to(dtype).to(device).contiguous().view(self.H, self.dv, self.R).transpose(1, 2)
        self.w_o = fetch("o").to(dtype).to(device).contiguous()
        # frequencies as the rotary part makes them (float64, the scaling's ramp, rounded once)
        rope = build_part("position", _PartSpec("rope_computed", {
            "rotary_dim": self.rot_dims, "theta": self.rot_base, "layout": "interleaved",
            "scaling": self.rot_scaling if self.rot_dims else None}))
        freq = rope.frequencies()
        self.amplitude = float(rope.amplitude)
        self.freq = (freq.to(torch.float32) if freq.numel() else torch.zeros(1)).to(device).contiguous()

    def weight_bytes(self) -> int:
        ts = [self.w_in, self.w_uk, self.w_uv_t, self.w_o, self.w_uq]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self):
        return PagedKVNeed(1, self.R + self.r, self.window, value_head_dim=0)

    def kernel_libraries(self):
        libs = ["core", "latent_attn"]
        if self.w_in is not None and self.w_in.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    # Prompt portions of at least this many tokens go through library products (scores and weighted sums of a
    # block of queries against the run of cached rows they see); shorter ones and single tokens go to the kernel
    # that walks each query's keys itself.
    PRODUCT_MIN_TOKENS = 32
    QUERY_BLOCK = 256

    def forward(self, x, step, cache):
        n, dev, H, d, r, R = x.shape[0], x.device, self.H, self.d, self.r, self.R
        proj = ops.linear(x, self.w_in)
        qrows = proj
        if self.q_rank is not None:          # the queries' own latent: norm, then the second product
            cq = torch.empty((n, self.q_rank), dtype=x.dtype, device=dev)
            ops.rmsnorm(cq, proj[:, :self.q_rank], self.q_norm_w, self.eps)
            qrows = ops.linear(cq, self.w_uq)
        q_full = torch.empty((n, H, R + r), dtype=x.dtype, device=dev)
        ops.latent_prepare(proj, 0, self.kv_off, self.norm_w, self.eps, self.freq, self.rot_dims, step.positions,
                           cache.slot_map if cache.writable else None, cache.k, q_full, H, d, r, R, step.status,
                           amplitude=self.amplitude, q=qrows)
        # queries into the latent space: a_h = Uk_h^T q_h, written in front of the rotated parts
        q_plain = qrows[:, :H * (d + r)].view(n, H, d + r)[:, :, :d].permute(1, 0, 2)         # [H, n, d]
        ops.batched_heads(q_plain, self.w_uk, out=q_full[:, :, :R].permute(1, 0, 2))            # [H, n, R]
        lat = torch.empty((n, H, R), dtype=x.dtype, device=dev)
        self.attend(lat, q_full, step, cache)
        heads = torch.empty((n, H * self.dv), dtype=x.dtype, device=dev)
        ops.batched_heads(lat.permute(1, 0, 2), self.w_uv_t, out=heads.view(n, H, self.dv).permute(1, 0, 2))
        return ops.linear(heads, self.w_o)

    def _splits(self, n, step, device):
        """How many CTAs share a query's keys (a CTA takes a query's 8 heads, 16 on tensor cores), and how many tiles
        of 32 positions each takes: few queries with
        many keys (decode steps) are spread until the CTAs fill the device about twice (a tile is a chain of
        latencies, so a CTA with one or two tiles beats fewer CTAs with more).
        The plan is made for the longest run of keys any query of the step may see (a captured step: of its class
        of context lengths), so it does not depend on what else is in the batch beyond that bound."""
        longest = step.max_kv_len if self.window is None else min(step.max_kv_len, self.window)
        tiles = (longest + 31) // 32 + 1                       # (a run that starts inside a tile touches one more)
        group = ops.latent_attention_heads(self.w_o.dtype, self.R, self.r)
        ctas = n * ((self.H + group - 1) // group)
        nsplit = max(1, min(tiles, (2 * ops.sm_count(device)) // max(1, ctas), 16))
        return nsplit, (tiles + nsplit - 1) // nsplit

    def attend(self, lat, q_full, step, cache) -> None:
        n, H, R, r = q_full.shape[0], self.H, self.R, self.r
        args = (H, R, r, cache.page_size, self.window, self.scale)
        entries = None if getattr(step, "captured", False) else getattr(step, "entries", None)
        if entries is None or all(len(e.tokens) < self.PRODUCT_MIN_TOKENS for e in entries):
            ops.latent_attention(lat, q_full, cache.k, cache.block_table, step, 0, n, *args,
                                 *self._splits(n, step, lat.device), sink=self.sink_w)
            return
        t, run0 = 0, 0          # run0: first token of the current run of entries that go to the kernel
        for e, ctx in zip(entries, step.entry_ctx):
            q = len(e.tokens)
            if q >= self.PRODUCT_MIN_TOKENS:
                if t > run0:
                    ops.latent_attention(lat, q_full, cache.k, cache.block_table, step, run0, t - run0, *args,
                                         sink=self.sink_w)
                self._attend_by_products(lat, q_full, cache, step, e.slot, t, q, ctx)
                run0 = t + q
            t += q
        if n > run0:     # (padding entries of a captured step never come here: such a step has no host entries)
            ops.latent_attention(lat, q_full, cache.k, cache.block_table, step, run0, n - run0, *args,
                                 sink=self.sink_w)

    def _attend_by_products(self, lat, q_full, cache, step, slot, t0, count, ctx) -> None:
        """Tokens t0 .. t0 + count - 1 of the step: one request's positions ctx .. ctx + count - 1."""
        H, R, KD = self.H, self.R, self.R + self.r
        for b0 in range(0, count, self.QUERY_BLOCK):
            nb = min(self.QUERY_BLOCK, count - b0)
            p0 = ctx + b0
            first = max(0, p0 - self.window + 1) if self.window else 0
            # the run starts at a multiple of 8 positions and is 8 k rows long (zero rows around the cached ones):
            # widths that the library's fast kernels take
            lo = first // 8 * 8
            keys = torch.empty(((p0 + nb - lo + 7) // 8 * 8, KD), dtype=lat.dtype, device=lat.device)
            ops.latent_gather(keys, cache.k, cache.block_table, slot, lo, cache.page_size, step.status,
                              first=first, last=p0 + nb - 1)
            qb = q_full[t0 + b0:t0 + b0 + nb].view(nb * H, KD)
            scores = ops.linear(qb, keys, out_dtype=torch.float32)                       # [nb * H, keys]
            weights = torch.empty(scores.shape, dtype=lat.dtype, device=lat.device)
            ops.latent_masked_softmax(weights, scores, H, p0, lo, self.window, self.scale, sink=self.sink_w)
            ops.product(weights, keys[:, :R], out=lat[t0 + b0:t0 + b0 + nb].view(nb * H, R))


register_part("mixer", "latent_attention", LatentAttention)
