"""Typed configuration of the Qwen2 dense decoder, read from its config.json keys.

Parity: ``ModelConfig.from_hf`` (servelab/config.py:48-72) reads hidden_size,
num_hidden_layers, num_attention_heads, num_key_value_heads (default: heads),
head_dim (default: hidden // heads), intermediate_size, vocab_size,
rms_norm_eps, rope_theta (default 1e6), max_position_embeddings (default 4096),
tie_word_embeddings (default False), torch_dtype (default "float16") and
eos_token_id (default 0).  The q/k/v bias of the architecture is fixed by its
name (``ARCH_QKV_BIAS``, servelab/parallel/tp_model.py:29); the output
projection and the MLP have no bias (tp_model.py:46,60-65).

Differences on purpose: ``eos_token_id`` may be a list; ``max_position_embeddings``
is kept so that the engine can enforce it; the window keys
(use_sliding_window / sliding_window / max_window_layers), which the reference
does not read, select a windowed mixer for the upper layers; model types the
reference aliases to qwen2 without handling their differences (qwen3) are
rejected.  The reference drops every key it does not know (config.py:48-72); here a
key that would change the arithmetic is an error instead of wrong logits:
``rope_scaling`` other than null (no scaled rotation exists in this engine),
``attention_bias`` / ``mlp_bias`` / ``partial_rotary_factor`` / ``attn_logit_softcapping``
and the like with a value other than the architecture's, and any key that is on
neither the list of keys read nor the list of keys known to be harmless.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .specs import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                    RMSNormSpec, RotarySpec)

_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads",
             "intermediate_size", "vocab_size", "rms_norm_eps")


# keys this class reads
_READ = frozenset(_REQUIRED) | {
    "num_key_value_heads", "head_dim", "rope_theta", "max_position_embeddings",
    "tie_word_embeddings", "torch_dtype", "dtype", "eos_token_id", "hidden_act",
    "use_sliding_window", "sliding_window", "max_window_layers", "layer_types",
    "architectures", "model_type"}
# keys that do not change a forward pass of this engine (training, generation defaults,
# bookkeeping of the library that wrote the file)
_HARMLESS = frozenset({
    "attention_dropout", "use_cache", "bos_token_id", "pad_token_id", "initializer_range",
    "transformers_version", "_name_or_path", "use_mrope", "output_attentions",
    "output_hidden_states", "return_dict", "is_decoder", "is_encoder_decoder",
    "tie_encoder_decoder", "add_cross_attention", "chunk_size_feed_forward",
    "id2label", "label2id", "problem_type", "finetuning_task", "tokenizer_class",
    "prefix", "sep_token_id", "decoder_start_token_id", "task_specific_params",
    "torchscript", "pruned_heads"})
# keys that may only carry the value the architecture has anyway
_FIXED = {"attention_bias": (None,), "mlp_bias": (False, None), "partial_rotary_factor": (1.0, None),
          "attn_logit_softcapping": (None,), "final_logit_softcapping": (None,),
          "rope_scaling": (None,), "rope_parameters": (None,), "qk_norm": (False, None),
          "quantization_config": (None,)}


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names every problem."""


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    torch_dtype: str
    eos_token_ids: Tuple[int, ...]
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "Qwen2Config":
        problems = [f"missing key '{k}'" for k in _REQUIRED if k not in cfg]
        for key, allowed in _FIXED.items():
            if key in cfg and cfg[key] not in allowed:
                problems.append(f"'{key}' = {cfg[key]!r} is not supported (it changes the "
                                f"arithmetic; only {' / '.join(map(repr, allowed))} is taken)")
        unknown = sorted(k for k in cfg if k not in _READ and k not in _HARMLESS and k not in _FIXED)
        if unknown:
            problems.append("unknown key(s) " + ", ".join(repr(k) for k in unknown)
                            + " (neither read nor known to be harmless)")
        if problems:
            raise ConfigError("invalid Qwen2 config: " + "; ".join(problems))
        heads = int(cfg["num_attention_heads"])
        hidden = int(cfg["hidden_size"])
        eos = cfg.get("eos_token_id", 0)
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        layers = int(cfg["num_hidden_layers"])
        use_win = bool(cfg.get("use_sliding_window", False))
        out = cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads", heads)),
            head_dim=int(cfg.get("head_dim", hidden // max(heads, 1))),
            intermediate_size=int(cfg["intermediate_size"]),
            vocab_size=int(cfg["vocab_size"]),
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            rope_theta=float(cfg.get("rope_theta", 1000000.0)),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            torch_dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "float16"))),
            eos_token_ids=eos_ids,
            hidden_act=str(cfg.get("hidden_act", "silu")),
            use_sliding_window=use_win,
            sliding_window=(int(cfg["sliding_window"])
                            if use_win and cfg.get("sliding_window") is not None else None),
            max_window_layers=int(cfg.get("max_window_layers", layers)),
        )
        out.validate()
        kinds = cfg.get("layer_types")
        if kinds is not None:
            # a per-layer list of "full_attention" / "sliding_attention": it must say what
            # the window keys say, or one of the two would be ignored
            mine = ["sliding_attention" if out.layer_window(i) else "full_attention"
                    for i in range(layers)]
            if list(kinds) != mine:
                raise ConfigError("invalid Qwen2 config: 'layer_types' disagrees with "
                                  "use_sliding_window / sliding_window / max_window_layers")
        return out

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen2Config":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        p = []
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size",
                     "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                p.append(f"{name} must be positive, got {getattr(self, name)}")
        if not p:
            if self.num_attention_heads % self.num_key_value_heads:
                p.append(f"num_attention_heads ({self.num_attention_heads}) is not a multiple "
                         f"of num_key_value_heads ({self.num_key_value_heads})")
            if self.head_dim % 2:
                p.append(f"head_dim ({self.head_dim}) must be even for rotary positions")
        if self.rms_norm_eps <= 0:
            p.append(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            p.append(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            p.append(f"hidden_act '{self.hidden_act}' is not the architecture's SiLU")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            p.append("use_sliding_window needs a positive sliding_window")
        if p:
            raise ConfigError("invalid Qwen2 config: " + "; ".join(p))

    def to_dict(self) -> Dict[str, Any]:
        d = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": self.torch_dtype,
            "eos_token_id": (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                             else list(self.eos_token_ids)),
            "hidden_act": self.hidden_act, "use_sliding_window": self.use_sliding_window,
        }
        if self.use_sliding_window:
            d["sliding_window"] = self.sliding_window
            d["max_window_layers"] = self.max_window_layers
        return d

    # ------------------------------------------------------------ derived
    @property
    def num_query_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    # ----------------------------------------------- the model as plain data
    def to_model_spec(self) -> ModelSpec:
        """Spell the architecture out layer by layer (pre-norm block, biased
        q/k/v, bias-free o and MLP, full rotary, RMSNorm everywhere); order of
        the layer body: servelab/parallel/tp_model.py:121-134."""
        rotary = RotarySpec(head_dim=self.head_dim, rotary_dim=self.head_dim,
                            theta=self.rope_theta)
        norm = RMSNormSpec(dim=self.hidden_size, eps=self.rms_norm_eps)
        ff = GatedMLPSpec(hidden_size=self.hidden_size,
                          intermediate_size=self.intermediate_size, activation="silu")
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = AttentionSpec(
                hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                qkv_bias=True, out_bias=False, window=self.layer_window(i),
                position=rotary)
            layers.append(BlockSpec(kind="pre_norm", mixer=mixer, feed_forward=ff,
                                    mixer_norm=norm, ff_norm=norm))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, layers=tuple(layers),
            run_order=tuple(LayerRun(i) for i in range(self.num_hidden_layers)),
            final_norm=norm, tie_word_embeddings=self.tie_word_embeddings,
            max_position_embeddings=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids)
