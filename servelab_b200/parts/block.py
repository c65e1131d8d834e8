"""Arrangement of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += ff(norm2(x)) -- the order of the
reference's layer body (servelab/parallel/tp_model.py:125-133).  The stream x is
float32; an update that has not been added yet travels beside it so that the add
happens inside the next norm kernel.
"""

from __future__ import annotations

from ..ops.kernels import plain_unless
from .base import Block
from .registry import FEED_FORWARDS, MIXERS, NORMS, build_part, part_class, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self._build(spec, prefix, env)
        # a step of this block may be captured in a CUDA graph iff every part only
        # launches kernels whose arguments are device buffers of the step context
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in
                              (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward))

    @staticmethod
    def _members(spec, prefix):
        """(registry, spec, prefix) of the four parts; the names under the layer's prefix are
        the spec's, so the block knows no checkpoint's naming."""
        return ((NORMS, spec.mixer_norm, f"{prefix}.{spec.mixer_norm_name}"),
                (MIXERS, spec.mixer, f"{prefix}.{spec.mixer_name}"),
                (NORMS, spec.ff_norm, f"{prefix}.{spec.ff_norm_name}"),
                (FEED_FORWARDS, spec.feed_forward, f"{prefix}.{spec.feed_forward_name}"))

    def _build(self, spec, prefix, env):
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = (
            build_part(table, part, name, env) for table, part, name in self._members(spec, prefix))

    @classmethod
    def declare(cls, spec, prefix):
        out = []
        for table, part, name in cls._members(spec, prefix):
            out += part_class(table, part).declare(part, name)
        return out

    @classmethod
    def cache_request(cls, spec):
        return part_class(MIXERS, spec.mixer).cache_request(spec.mixer)

    def load(self, store):
        for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward):
            p.load(store)

    accepts_split_sum = True          # the incoming ``delta`` may be a SplitSum
    accepts_deferred_linear = True    # ... or a DeferredLinear

    def forward(self, ctx, resid, delta, cache, owns_cache):
        # An update may arrive in an unfinished form (the partial sums of a K-split product, a
        # product not launched yet), and a norm may return its rows in one (ScaledRows): a part
        # that does not say that it takes the form gets the plain tensor.
        x = self.mixer_norm.forward(ctx, resid, plain_unless(self.mixer_norm, delta))
        a = self.mixer.forward(ctx, plain_unless(self.mixer, x), cache, owns_cache)
        x = self.ff_norm.forward(ctx, resid, plain_unless(self.ff_norm, a))
        return resid, self.feed_forward.forward(ctx, plain_unless(self.feed_forward, x))
