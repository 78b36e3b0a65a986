"""Registries from a spec's ``kind`` to the class that implements it.

A new norm, position encoding, mixer, feed-forward or arrangement of a layer is a class registered here under a
new kind; the block and the decoder build whatever the specs name and know no kind themselves.
"""
from __future__ import annotations

from typing import Callable, Dict

_REGISTRIES: Dict[str, Dict[str, Callable]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}}


def _register(family: str, kind: str, factory: Callable, replace: bool = False) -> None:
    table = _REGISTRIES[family]
    if kind in table and not replace:
        raise KeyError(f"{family} kind {kind!r} is already registered")
    table[kind] = factory


def _build(family: str, spec, kind=None):
    table = _REGISTRIES[family]
    kind = spec.kind if kind is None else kind
    if kind not in table:
        raise KeyError(f"no {family} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind](spec)


def register_norm(kind, factory, replace=False):
    _register("norm", kind, factory, replace)


def register_position(kind, factory, replace=False):
    _register("position", kind, factory, replace)


def register_mixer(kind, factory, replace=False):
    _register("mixer", kind, factory, replace)


def register_feed_forward(kind, factory, replace=False):
    _register("feed_forward", kind, factory, replace)


def register_block(arrangement, factory, replace=False):
    """``arrangement``: the value of ``BlockSpec.arrangement`` that this class builds."""
    _register("block", arrangement, factory, replace)


def build_block(spec):
    return _build("block", spec, spec.arrangement)


def build_norm(spec):
    return _build("norm", spec)


def build_position(spec):
    return _build("position", spec)


def build_mixer(spec):
    return _build("mixer", spec)


def build_feed_forward(spec):
    return _build("feed_forward", spec)


def registered(family: str):
    return sorted(_REGISTRIES[family])
