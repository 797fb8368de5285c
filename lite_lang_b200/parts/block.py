"""Pre-norm arrangement: h += mixer(norm(h)); h += feed_forward(norm(h)).

``litelang/models/qwen2/layer/transformer_layer.py:46-77``.  The residual sums
are folded into the norm that follows them (one pass over the row instead of
two), which is why a block hands its last, not yet added, output on as ``delta``.
"""

from __future__ import annotations

from .base import Block, NormEntry, NormSplit, register_part


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


register_part("block", "pre_norm", PreNormBlock)
