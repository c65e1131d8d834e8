"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no experts, no routing
(servelab/parallel/tp_model.py:60-68 in the reference).  gate and up are fused
into one [2I, h] matrix at load so that one product feeds the activation kernel;
when I allows it their rows alternate in runs of 64, so that a 128-row tile of the
decode-step product holds 64 gates with their ups and applies the activation itself.
"""

from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops.linear import gated_linear, linear
from ..weights.source import BIAS, MATRIX, TensorDecl
from .base import FeedForward
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    accepts_scaled_rows = True        # ``x`` may be ScaledRows: the gate|up product applies 1 / rms

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation {spec.activation!r} has no kernel (silu only)")
        if spec.bias:
            raise ValueError("gated_mlp: biases are not supported")

    @classmethod
    def declare(cls, spec, prefix):
        h, i = spec.hidden_size, spec.intermediate_size
        return [TensorDecl(f"{prefix}.{spec.gate_name}.weight", (i, h), MATRIX),
                TensorDecl(f"{prefix}.{spec.up_name}.weight", (i, h), MATRIX),
                TensorDecl(f"{prefix}.{spec.down_name}.weight", (h, i), MATRIX)]

    def load(self, store):
        gate = store.get(f"{self.prefix}.{self.spec.gate_name}.weight")
        up = store.get(f"{self.prefix}.{self.spec.up_name}.weight")
        inter, h = gate.shape
        self.block = K.SWIGLU_BLOCK if inter % K.SWIGLU_BLOCK == 0 else 0
        if self.block:
            b = self.block
            self.w_gate_up = torch.stack([gate.view(inter // b, b, h), up.view(inter // b, b, h)],
                                         dim=1).reshape(2 * inter, h).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0)
        self.w_down = store.get(f"{self.prefix}.{self.spec.down_name}.weight")

    def forward(self, ctx, x):
        act = gated_linear(x, self.w_gate_up, self.block)
        return linear(act, self.w_down, consumer="norm")
