"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no experts, no routing
(servelab/parallel/tp_model.py:60-68 in the reference).  gate and up are fused
into one [2I, h] matrix at load so that one product feeds the activation kernel.
"""

from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.source import BIAS, MATRIX, TensorDecl
from .base import FeedForward
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation {spec.activation!r} has no kernel (silu only)")
        if spec.bias:
            raise ValueError("gated_mlp: biases are not supported")

    @classmethod
    def declare(cls, spec, prefix):
        h, i = spec.hidden_size, spec.intermediate_size
        return [TensorDecl(prefix + ".gate_proj.weight", (i, h), MATRIX),
                TensorDecl(prefix + ".up_proj.weight", (i, h), MATRIX),
                TensorDecl(prefix + ".down_proj.weight", (h, i), MATRIX)]

    def load(self, store):
        self.w_gate_up = store.cat([self.prefix + ".gate_proj.weight",
                                    self.prefix + ".up_proj.weight"])
        self.w_down = store.get(self.prefix + ".down_proj.weight")

    def matrices(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, ctx, x):
        gu = linear(x, self.w_gate_up)
        act = torch.empty((x.shape[0], self.spec.intermediate_size), dtype=x.dtype, device=x.device)
        K.swiglu(gu, act)
        return linear(act, self.w_down, consumer="norm")
