"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` (the architecture's own keys) and
``model.safetensors`` with every tensor the model declares, under the
checkpoint's names.  Distributions: matrices and biases N(0, 0.02^2), norm
weights 1 + N(0, 0.1^2).  The reference's counterpart builds a tiny random
checkpoint for its tests (tests/helpers_tiny_model.py:7-56) with N(0, 0.05^2)
matrices, zero biases and unit norms; non-trivial biases and norm weights are
used here so that a dropped bias or norm weight changes the logits.
"""

from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors
from .source import TABLE, RandomSource


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.float32,
                       std: float = 0.02, norm_std: float = 0.1, std_of=None) -> str:
    """``config`` is a typed architecture config (``to_dict``/``to_model_spec``);
    ``std_of`` maps parts of tensor names to standard deviations of their own
    (``RandomSource``)."""
    from ..models.causal_lm import declare_tensors  # parts declare their tensors

    os.makedirs(folder, exist_ok=True)
    decls = declare_tensors(config.to_model_spec())
    src = RandomSource(decls, seed, std=std, norm_std=norm_std, dtype=dtype, std_of=std_of)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(
        os.path.join(folder, "model.safetensors"),
        [(d.name, tuple(d.shape), torch.int32 if d.role == TABLE else dtype) for d in decls],
        src.read, metadata={"format": "pt", "seed": seed})
    return folder
