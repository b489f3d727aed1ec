"""Registries of part classes, keyed by the ``kind`` of their spec.

A part class is registered under a category (mixer, ffn, norm, position, block) and a kind;
``build(category, spec, **kw)`` constructs it.  A new mixer, feed-forward, norm, position
encoding or block arrangement is a class plus one ``register`` call; nothing else in the
framework names part kinds.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

CATEGORIES = ("mixer", "ffn", "norm", "position", "block")
_PARTS: Dict[Tuple[str, str], Callable] = {}


def register(category: str, kind: str, cls=None):
    """``register("mixer", "attention", Attention)`` or as a decorator without ``cls``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def deco(c):
        _PARTS[(category, kind)] = c
        return c

    return deco(cls) if cls is not None else deco


def registered(category: str):
    return sorted(k for c, k in _PARTS if c == category)


def build(category: str, spec, **kw):
    kind = getattr(spec, "kind", None)
    cls = _PARTS.get((category, kind))
    if cls is None:
        raise KeyError(f"no {category} registered for kind {kind!r}; registered: {registered(category)}")
    return cls(spec, **kw)
