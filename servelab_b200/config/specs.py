"""Architecture-neutral description of a model as data.

A model is a list of *layers*, each a block that names its parts (mixer,
feed-forward, norms) by registry kind together with their sizes and constants,
plus a *run order*: the sequence in which layers execute, which may name a layer
twice or let a run read the cache that an earlier run filled.  Nothing in here knows any
model family; the family's config class (for example ``Qwen2Config``) translates
its own ``config.json`` keys into these specs.

The specs are frozen dataclasses so they can be hashed, compared and printed.
A spec's ``kind`` selects the implementation from the part registries in
``servelab_b200.parts.registry``; new kinds are added by registering a part
there, never by editing this file.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description: ``kind`` is the registry key."""
    kind: str


# ----------------------------------------------------------------- positions
@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding over the first ``rotary_dim``
    elements of each head (``rotary_dim == head_dim`` for a full rotation)."""
    kind: str = "rotary"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: str = "none"


# --------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    kind: str = "rmsnorm"
    dim: int = 0
    eps: float = 1e-6


# -------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` is None for attention over all earlier keys, else the number of
    most recent keys (the query's own included) a query may see.
    """
    kind: str = "paged_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None => head_dim ** -0.5
    position: PartSpec = field(default_factory=NoPositionSpec)
    # checkpoint names of the projections under the mixer's prefix (data, like the sizes:
    # an architecture with the same arithmetic and other names changes these, not the part)
    q_name: str = "q_proj"
    k_name: str = "k_proj"
    v_name: str = "v_proj"
    o_name: str = "o_proj"
    position_name: str = "rotary_emb"


# -------------------------------------------------------------- feed-forward
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down(act(gate(x)) * up(x)) with a dense (expert-free) gate/up/down."""
    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    bias: bool = False
    gate_name: str = "gate_proj"           # checkpoint names under the feed-forward's prefix
    up_name: str = "up_proj"
    down_name: str = "down_proj"


# --------------------------------------------------------------------- block
@dataclass(frozen=True)
class BlockSpec(PartSpec):
    """One layer: how a mixer, a feed-forward and their norms are arranged.
    ``pre_norm`` is x += mixer(norm1(x)); x += ff(norm2(x))."""
    kind: str = "pre_norm"
    mixer: PartSpec = None
    feed_forward: PartSpec = None
    mixer_norm: PartSpec = None
    ff_norm: PartSpec = None
    # checkpoint names of the four parts under the layer's prefix
    mixer_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn"
    ff_norm_name: str = "post_attention_layernorm"
    feed_forward_name: str = "mlp"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``layer``      index into ``ModelSpec.layers`` (weights and parts).  A layer may
                   be named by several runs; they share its weights, and each run
                   that owns a cache gets one of its own.
    ``cache_of``   index of an EARLIER RUN whose cache this run reads instead of
                   owning one: such a run writes no keys, values or state.  None
                   means the run owns (and fills) its cache.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build a model; no family-specific keys."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[BlockSpec, ...]
    run_order: Tuple[LayerRun, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = ()
    # a position encoding that acts on the embedded tokens (learned or sinusoidal
    # absolute positions); encodings that act inside a mixer belong to its spec
    embedding_position: PartSpec = field(default_factory=NoPositionSpec)
    embedding_position_prefix: str = "model.embed_positions"
    # checkpoint naming: prefix of layer i is layer_prefix.format(i)
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm"
    layer_prefix: str = "model.layers.{}"
    # checkpoint tensors that may be present and are ignored
    ignored_suffixes: Tuple[str, ...] = ("rotary_emb.inv_freq",)
    # arithmetic around the layers that some architectures have; None: not applied
    embedding_scale: Optional[float] = None      # embedded tokens are multiplied by it
    logit_scale: Optional[float] = None          # logits are multiplied by it ...
    logit_softcap: Optional[float] = None        # ... and then become cap * tanh(logits / cap)
