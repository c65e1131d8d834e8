"""The one registry from an architecture's name to its model.

``config.json`` names its architecture in ``architectures[0]`` (falling back to
``model_type``).  An entry supplies the typed config class of that architecture;
the config class turns itself into a ``ModelSpec`` from which the generic
``CausalLM`` is built, so "the model of an architecture" is data plus the parts
it names.  The reference has no registry: its engine hard-codes one decoder
class and a ``model_type`` whitelist (servelab/config.py:50-54,
servelab/engine/engine.py:72-85); unknown names raise the same
"unsupported architecture" ValueError here.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple

from .specs import ModelSpec

_ARCHITECTURES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_cls: type, model_type: str = "") -> None:
    """``config_cls`` needs ``from_dict(dict)``, ``to_dict()`` and
    ``to_model_spec() -> ModelSpec``."""
    _ARCHITECTURES[name] = config_cls
    if model_type:
        _MODEL_TYPES[model_type] = name


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(cfg: Dict[str, Any]) -> str:
    archs = cfg.get("architectures") or []
    if archs:
        name = archs[0]
        if name in _ARCHITECTURES:
            return name
        raise ValueError(f"unsupported architecture: {name} "
                         f"(registered: {', '.join(registered_architectures())})")
    mtype = cfg.get("model_type")
    if mtype in _MODEL_TYPES:
        return _MODEL_TYPES[mtype]
    raise ValueError(f"unsupported architecture: model_type={mtype!r} "
                     f"(registered: {', '.join(registered_architectures())})")


def config_from_dict(cfg: Dict[str, Any]):
    return _ARCHITECTURES[resolve_architecture(cfg)].from_dict(cfg)


def load_config(folder: str):
    """Typed config of the model folder, its class chosen by config.json."""
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in model folder {folder!r}")
    with open(path) as f:
        return config_from_dict(json.load(f))


def model_spec_from_config(config) -> ModelSpec:
    return config.to_model_spec()
