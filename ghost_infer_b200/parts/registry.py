"""Registries from a part's kind (the name a `PartSpec` carries) to its class."""
from __future__ import annotations

from typing import Callable, Dict

_KINDS = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRIES: Dict[str, Dict[str, type]] = {k: {} for k in _KINDS}


def register(family: str, kind: str, cls: type = None, *, replace: bool = False):
    """`register("mixer", "gqa_attention", GqaAttention)`, or as a decorator without `cls`."""
    if family not in _REGISTRIES:
        raise ValueError(f"unknown family of parts {family!r} (known: {', '.join(_KINDS)})")

    def put(c: type) -> type:
        if kind in _REGISTRIES[family] and not replace:
            raise ValueError(f"{family} \"{kind}\" is already registered")
        _REGISTRIES[family][kind] = c
        return c

    return put if cls is None else put(cls)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def lookup(family: str, kind: str) -> type:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES.get(family, {}))) or "none"
        raise KeyError(f"no {family} of kind \"{kind}\" is registered (registered: {known})") from None


def registered(family: str) -> tuple:
    return tuple(sorted(_REGISTRIES[family]))
