"""Models: the generic causal LM assembled from a ModelSpec."""

from .causal_lm import CausalLM, declare_tensors

__all__ = ["CausalLM", "declare_tensors"]
