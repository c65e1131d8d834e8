"""The generic causal language model: embedding, blocks in run order, final norm,
LM head -- built from a ``ModelSpec`` and the part registries.

``declare_tensors(spec)`` lists every checkpoint tensor the model needs (without
building anything), ``CausalLM.load`` fills the parts from a checked source, and
``forward`` runs the tokens of one step and returns float32 logits at the wanted
rows.  Order of operations: servelab/parallel/tp_model.py:121-134 (embed, layers,
final norm) and :112-119 (LM head; tied weights reuse the embedding table); the
optional embedding scale and logit scale / soft cap of the spec are applied where
architectures that have them apply them (Qwen2 has none); rows
are selected before the final norm here, which gives the same result because the
norm acts per row (the reference norms all rows first, servelab/engine/
engine.py:217-218).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..parts import BLOCKS, NORMS, POSITIONS, BuildEnv, LayerCache, build_part, part_class
from ..weights.source import MATRIX, TensorDecl, WeightSource
from ..weights.store import WeightStore


def declare_tensors(spec: ModelSpec) -> List[TensorDecl]:
    out = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), MATRIX)]
    out += part_class(POSITIONS, spec.embedding_position).declare(spec.embedding_position,
                                                                  spec.embedding_position_prefix)
    for i, block in enumerate(spec.layers):
        out += part_class(BLOCKS, block).declare(block, spec.layer_prefix.format(i))
    out += part_class(NORMS, spec.final_norm).declare(spec.final_norm, spec.final_norm_prefix)
    if not spec.tie_word_embeddings:
        out.append(TensorDecl(spec.lm_head_name, (spec.vocab_size, spec.hidden_size), MATRIX))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        for i, run in enumerate(spec.run_order):
            if not 0 <= run.layer < len(spec.layers):
                raise ValueError(f"run order names layer {run.layer}, model has {len(spec.layers)}")
            if run.cache_of is not None and (
                    not 0 <= run.cache_of < i or spec.run_order[run.cache_of].cache_of is not None):
                raise ValueError(f"run {i} reads the cache of run {run.cache_of}, which must be "
                                 f"an earlier run that owns a cache")
        self.blocks = [build_part(BLOCKS, b, spec.layer_prefix.format(i), env)
                       for i, b in enumerate(spec.layers)]
        self.final_norm = build_part(NORMS, spec.final_norm, spec.final_norm_prefix, env)
        self.embedding_position = build_part(POSITIONS, spec.embedding_position,
                                             spec.embedding_position_prefix, env)
        self.embed_tokens: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------ caches
    def cache_requests(self) -> List[Optional[object]]:
        """Per run of the run order, what its mixer asks of the cache; None for
        runs that read an earlier run's cache."""
        return [part_class(BLOCKS, self.spec.layers[run.layer]).cache_request(
                    self.spec.layers[run.layer]) if run.cache_of is None else None
                for run in self.spec.run_order]

    # ----------------------------------------------------------- weights
    def load(self, source: WeightSource) -> None:
        optional = (self.spec.lm_head_name,) if self.spec.tie_word_embeddings else ()
        store = WeightStore(source, declare_tensors(self.spec), self.env.dtype, self.env.device,
                            ignored_suffixes=self.spec.ignored_suffixes, optional=optional)
        self.embed_tokens = store.get(self.spec.embed_name)
        self.embedding_position.load(store)
        for b in self.blocks:
            b.load(store)
        self.final_norm.load(store)
        self.lm_head = (self.embed_tokens if self.spec.tie_word_embeddings
                        else store.get(self.spec.lm_head_name))

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def walk(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
                elif hasattr(v, "spec") and hasattr(v, "env"):
                    walk(v)
        for b in self.blocks:
            walk(b)
        walk(self.final_norm)
        for t in (self.embed_tokens, self.lm_head):
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ----------------------------------------------------------- forward
    def forward(self, ctx, caches: Dict[int, LayerCache]) -> torch.Tensor:
        """Run the step's tokens; ``caches`` maps a run's index to its cache.
        Returns logits [wanted rows, vocab] float32."""
        T = ctx.num_tokens
        resid = torch.empty((T, self.spec.hidden_size), dtype=torch.float32, device=self.env.device)
        K.embedding(ctx.token_ids, self.embed_tokens, resid,
                    1.0 if self.spec.embedding_scale is None else self.spec.embedding_scale)
        self.embedding_position.apply_to_embedding(ctx, resid)
        delta = None
        for i, run in enumerate(self.spec.run_order):
            owner = i if run.cache_of is None else run.cache_of
            block = self.blocks[run.layer]
            # (an update may travel as the partial sums of a K-split product; a block that
            # does not say it accepts that form gets the plain tensor)
            resid, delta = block.forward(ctx, resid, K.plain_unless(block, delta), caches[owner],
                                         run.cache_of is None)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.env.device)
        x = self.final_norm.forward(ctx, resid, K.plain_unless(self.final_norm, delta),
                                    out_rows=ctx.logit_rows)
        logits = linear(x, self.lm_head, out_dtype=torch.float32)
        if self.spec.logit_scale is not None or self.spec.logit_softcap is not None:
            K.logit_transform(logits, 1.0 if self.spec.logit_scale is None else self.spec.logit_scale,
                              self.spec.logit_softcap or 0.0)
        return logits
