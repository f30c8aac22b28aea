"""Arrangements of a layer's parts.

Pre-norm: h += mixer(norm(h)); h += feed_forward(norm(h)).

``litelang/models/qwen2/layer/transformer_layer.py:46-77``.  The residual sums
are folded into the norm that follows them (one pass over the row instead of
two), which is why a block hands its last, not yet added, output on as ``delta``.
"""

from __future__ import annotations

from .. import ops
from .base import Block, NormEntry, NormSplit, ResidualCopy, register_part


class PreNormBlock(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, h, delta, step, caches):
        cache = caches["mixer"]
        x = self.mixer_norm.add_forward(h, delta)
        # a part that can add its output to h in its last product (portions of prompts) returns None; one that
        # can also leave the norm after it to the product that follows (decode steps) returns a NormSplit
        into = None
        if self.mixer.splits_norm and self.feed_forward.takes_norm_split:
            params = self.feed_forward_norm.split_params()
            if params is not None:
                into = NormEntry(params[0], params[1], self.feed_forward.accepts_norm_split)
        if into is not None:
            a = self.mixer.forward(x, step, cache, residual=h, into_norm=into)
        elif self.mixer.accumulates:
            a = self.mixer.forward(x, step, cache, residual=h)
        else:
            a = self.mixer.forward(x, step, cache)
        x = a if isinstance(a, NormSplit) else self.feed_forward_norm.add_forward(h, a)
        f = (self.feed_forward.forward(x, step, residual=h) if self.feed_forward.accumulates
             else self.feed_forward.forward(x, step))
        return h, f


class PreNormMixerOnlyBlock(Block):
    """The pre-norm arrangement of a layer without a feed-forward: h += mixer(norm(h))."""

    roles = {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, h, delta, step, caches):
        x = self.mixer_norm.add_forward(h, delta)
        return h, self.mixer.forward(x, step, caches["mixer"])


class ParallelBlock(Block):
    """Parallel arrangement: with n = norm(h), h += mixer(n) + feed_forward(n).  One norm; both parts read
    its output.  Their outputs are handed on together and added (to each other, then to the residual
    stream) inside the next norm."""

    roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, h, delta, step, caches):
        x = self.norm.add_forward(h, delta)
        a = self.mixer.forward(x, step, caches["mixer"])
        f = self.feed_forward.forward(x, step)
        return h, (a, f)


class ParallelMixerOnlyBlock(Block):
    """The parallel arrangement of a layer without a feed-forward: h += mixer(norm(h))."""

    roles = {"norm": "norm", "mixer": "mixer"}

    def forward(self, h, delta, step, caches):
        x = self.norm.add_forward(h, delta)
        return h, self.mixer.forward(x, step, caches["mixer"])


class OutputNormBlock(Block):
    """Norm on the sublayers' outputs: h += norm(mixer(h)); h += norm(feed_forward(h)).  The sublayers read the
    float32 residual stream itself, rounded to the engine's dtype; that copy is made by the norm's pass over the
    residual and handed on to the next block in the place of a pending output (``ResidualCopy``)."""

    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}

    @staticmethod
    def _operand(h, delta, dtype):
        if isinstance(delta, ResidualCopy):
            return delta.rows
        if delta is not None:
            raise TypeError("a block with norms on its sublayers' outputs cannot take a pending output")
        return ops.round_rows(h, dtype)

    def forward(self, h, delta, step, caches):
        x = self._operand(h, delta, self.mixer_norm.out_dtype)
        x = self.mixer_norm.add_into(h, self.mixer.forward(x, step, caches["mixer"]))
        x = self.feed_forward_norm.add_into(h, self.feed_forward.forward(x, step))
        return h, ResidualCopy(x)


class OutputNormMixerOnlyBlock(OutputNormBlock):
    """The same arrangement for a layer without a feed-forward: h += norm(mixer(h))."""

    roles = {"mixer": "mixer", "mixer_norm": "norm"}

    def forward(self, h, delta, step, caches):
        x = self._operand(h, delta, self.mixer_norm.out_dtype)
        x = self.mixer_norm.add_into(h, self.mixer.forward(x, step, caches["mixer"]))
        return h, ResidualCopy(x)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "pre_norm_mixer_only", PreNormMixerOnlyBlock)
register_part("block", "output_norm", OutputNormBlock)
register_part("block", "output_norm_mixer_only", OutputNormMixerOnlyBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "parallel_mixer_only", ParallelMixerOnlyBlock)
