"""Arrangement of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += ff(norm2(x)) -- the order of the
reference's layer body (servelab/parallel/tp_model.py:125-133).  The stream x is
float32; an update that has not been added yet travels beside it so that the add
happens inside the next norm kernel.
"""

from __future__ import annotations

from ..ops.kernels import plain_unless
from .base import Block
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, build_part, part_class,
                       register_block)


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self._build(spec, prefix, env)
        # a step of this block may be captured in a CUDA graph iff every part only
        # launches kernels whose arguments are device buffers of the step context
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in
                              (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward))

    def _build(self, spec, prefix, env):
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, prefix + ".input_layernorm", env)
        self.mixer = build_part(MIXERS, spec.mixer, prefix + ".self_attn", env)
        self.ff_norm = build_part(NORMS, spec.ff_norm, prefix + ".post_attention_layernorm", env)
        self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, prefix + ".mlp", env)

    @classmethod
    def declare(cls, spec, prefix):
        return (part_class(NORMS, spec.mixer_norm).declare(spec.mixer_norm, prefix + ".input_layernorm")
                + part_class(MIXERS, spec.mixer).declare(spec.mixer, prefix + ".self_attn")
                + part_class(NORMS, spec.ff_norm).declare(spec.ff_norm,
                                                          prefix + ".post_attention_layernorm")
                + part_class(FEED_FORWARDS, spec.feed_forward).declare(spec.feed_forward,
                                                                       prefix + ".mlp"))

    @classmethod
    def cache_request(cls, spec):
        return part_class(MIXERS, spec.mixer).cache_request(spec.mixer)

    def load(self, store):
        for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward):
            p.load(store)

    def matrices(self):
        return self.mixer.matrices() + self.feed_forward.matrices()

    accepts_split_sum = True          # the incoming ``delta`` may be a SplitSum
    accepts_deferred_linear = True    # ... or a product that has not run

    @staticmethod
    def _norm(norm, consumer, ctx, resid, delta):
        """The norm before ``consumer``.  An update may arrive unfinished (partial sums of
        a K-split product, a product that has not run); a norm that does not take the
        form gets the plain tensor.  A norm that can leave its own result unfinished does
        so if the consumer takes it."""
        delta = plain_unless(norm, delta)
        if getattr(norm, "returns_lazy_norm", False) and getattr(consumer, "accepts_lazy_norm", False):
            return norm.forward(ctx, resid, delta, lazy_ok=True)
        return norm.forward(ctx, resid, delta)

    def forward(self, ctx, resid, delta, cache, owns_cache):
        x = self._norm(self.mixer_norm, self.mixer, ctx, resid, delta)
        a = self.mixer.forward(ctx, x, cache, owns_cache)
        x = self._norm(self.ff_norm, self.feed_forward, ctx, resid, a)
        return resid, self.feed_forward.forward(ctx, x)
