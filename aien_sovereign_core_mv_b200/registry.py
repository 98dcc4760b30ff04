"""Registries: one from an architecture's name to its builder, one per kind of part.

An *architecture builder* turns a parsed ``config.json`` into a typed configuration and a
:class:`~.config.spec.ModelSpec`.  A *part factory* turns a ``PartSpec`` into a part object.
New entries are added from outside the package with the ``register_*`` decorators; the
framework's files do not change (the tests register a toy mixer this way).
"""
from __future__ import annotations

from typing import Any, Callable, Dict

_ARCHITECTURES: Dict[str, Callable[..., Any]] = {}
_PARTS: Dict[str, Dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def register_architecture(name: str):
    """Decorator: ``builder(raw_config: dict, generation_config: dict|None, strict: bool)
    -> (typed_config, ModelSpec)``."""

    def deco(fn):
        _ARCHITECTURES[name] = fn
        return fn

    return deco


def architecture_names():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError(
            f"unsupported architecture {name!r}: registered are {architecture_names()}"
        ) from None


def _register(family: str, kind: str):
    def deco(factory):
        _PARTS[family][kind] = factory
        return factory

    return deco


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_block(kind: str):
    return _register("block", kind)


def register_embedding(kind: str):
    return _register("embedding", kind)


def register_head(kind: str):
    return _register("head", kind)


def part_factory(family: str, kind: str):
    """The registered class (or function) itself: what a block declares about itself, such as
    the norm slots it wants, is read from it before anything is built."""
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise KeyError(
            f"no {family} part of kind {kind!r}: registered are {sorted(_PARTS[family])}"
        ) from None


def make_part(family: str, kind: str, *args, **kwargs):
    return part_factory(family, kind)(*args, **kwargs)


def part_kinds(family: str):
    return sorted(_PARTS[family])
