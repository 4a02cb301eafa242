"""Registries from a part's kind to the class that builds it.

A model names its parts by kind (`PartSpec.kind`); these tables turn the kind
into a class.  Anyone, a test included, may add a kind with the `register_*`
functions; nothing else in the framework has to change for the new part to be
built, given a cache, and stepped.
"""

from __future__ import annotations

from typing import Any, Callable

MIXERS: dict[str, Callable[..., Any]] = {}
FEED_FORWARDS: dict[str, Callable[..., Any]] = {}
NORMS: dict[str, Callable[..., Any]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., Any]] = {}
BLOCKS: dict[str, Callable[..., Any]] = {}
EMBEDDINGS: dict[str, Callable[..., Any]] = {}
HEADS: dict[str, Callable[..., Any]] = {}

_TABLES = {
    "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS,
    "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS,
}


def _register(table: dict, what: str, kind: str, factory: Callable[..., Any], replace: bool) -> None:
    if kind in table and not replace and table[kind] is not factory:
        raise ValueError(f"{what} kind {kind!r} is already registered")
    table[kind] = factory


def register_mixer(kind: str, factory, replace: bool = False) -> None:
    _register(MIXERS, "mixer", kind, factory, replace)


def register_feed_forward(kind: str, factory, replace: bool = False) -> None:
    _register(FEED_FORWARDS, "feed-forward", kind, factory, replace)


def register_norm(kind: str, factory, replace: bool = False) -> None:
    _register(NORMS, "norm", kind, factory, replace)


def register_position_encoding(kind: str, factory, replace: bool = False) -> None:
    _register(POSITION_ENCODINGS, "position encoding", kind, factory, replace)


def register_block(kind: str, factory, replace: bool = False) -> None:
    _register(BLOCKS, "block", kind, factory, replace)


def register_embedding(kind: str, factory, replace: bool = False) -> None:
    _register(EMBEDDINGS, "embedding", kind, factory, replace)


def register_head(kind: str, factory, replace: bool = False) -> None:
    _register(HEADS, "head", kind, factory, replace)


def build_part(role: str, spec, **context):
    """Instantiate `spec` (a PartSpec) from the table for `role`; `context` carries dtype and device."""
    table = _TABLES[role]
    if spec.kind not in table:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered; known: {sorted(table)}")
    return table[spec.kind](**dict(spec.params), **context)
