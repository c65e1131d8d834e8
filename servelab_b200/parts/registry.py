"""Registries from a spec's ``kind`` to the part that implements it.

Adding a mixer, feed-forward, norm, position encoding or block arrangement is
``register_<family>("kind")(cls)`` plus a spec dataclass whose ``kind`` names it;
nothing else in the package changes.
"""

from __future__ import annotations

from typing import Callable, Dict

from .base import BuildEnv

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}


def _register(table: Dict[str, type], family: str) -> Callable[[str], Callable[[type], type]]:
    def by_kind(kind: str):
        def deco(cls: type) -> type:
            table[kind] = cls
            return cls
        return deco
    by_kind.__name__ = f"register_{family}"
    return by_kind


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed_forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position")
register_block = _register(BLOCKS, "block")


def part_class(table: Dict[str, type], spec) -> type:
    try:
        return table[spec.kind]
    except KeyError:
        raise KeyError(f"no part registered for kind {spec.kind!r} "
                       f"(known: {', '.join(sorted(table))})") from None


def build_part(table: Dict[str, type], spec, prefix: str, env: BuildEnv):
    return part_class(table, spec)(spec, prefix, env)
