"""Position encodings.

``rotary``: rotate-half rotary embedding; inv_freq_i = theta^(-2i/rotary_dim) in
float32, as the reference builds it (servelab/parallel/tp_model.py:94-95; the
buffer is never cast to the model dtype here, unlike tp_model.py:96-97).  The
rotation itself is fused into the mixer's q/k kernel, which asks this part for
its table.  ``none``: no position information.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position


@register_position("rotary")
class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        rd = spec.rotary_dim or spec.head_dim
        if rd % 2 or rd > spec.head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and <= head_dim {spec.head_dim}")
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        self.rotary_dim = rd
        self.inv_freq = inv_freq.to(env.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True
