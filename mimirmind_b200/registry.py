"""Registries: architecture name → model builder, part kind → part class.

The reference maps an architecture string to a backend object in one switch and
fails naming the string when it is unknown (src/runtime/arch/ArchBackend.cpp:14-55;
src/runtime/InferenceEngine.cpp:1321-1328), with a pure-name predicate for tests
(src/runtime/arch/ArchBackend.hpp:231-235).  Here both levels are open tables so that
another mixer, feed-forward, norm, position encoding, block arrangement or whole
architecture is added by registering it, not by editing engine files.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message; keep it readable
        return self.args[0] if self.args else ""


class _Table:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Any] = {}

    def register(self, name: str, item: Any = None, *, replace: bool = False):
        def put(obj):
            if name in self._items and not replace and self._items[name] is not obj:
                raise RegistryError(f"{self.what} '{name}' is already registered")
            self._items[name] = obj
            return obj

        if item is None:
            return put  # decorator form
        return put(item)

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> Any:
        try:
            return self._items[name]
        except KeyError:
            known = ", ".join(sorted(self._items)) or "(none)"
            raise RegistryError(f"unknown {self.what} '{name}'; known: {known}") from None

    def names(self) -> List[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


# architecture name (config.json "architectures"[0]) → ArchitectureEntry
ARCHITECTURES = _Table("architecture")
# part kinds
MIXERS = _Table("mixer")
FEED_FORWARDS = _Table("feed-forward")
NORMS = _Table("norm")
POSITION_ENCODINGS = _Table("position encoding")
BLOCKS = _Table("block arrangement")
EMBEDDINGS = _Table("embedding")
HEADS = _Table("output head")
# the tables by the category a PartSpec may name (a layer's extra parts say which table holds their kind)
CATEGORIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS, "block": BLOCKS,
              "embedding": EMBEDDINGS, "head": HEADS}


def part_class(spec) -> Any:
    """The class of a PartSpec that names its category."""
    try:
        table = CATEGORIES[spec.category]
    except KeyError:
        raise RegistryError(f"part of kind '{spec.kind}' names the category '{spec.category}'; known: {', '.join(sorted(CATEGORIES))}") from None
    return table.get(spec.kind)


class ArchitectureEntry:
    """What an architecture registers: how to parse its config and how to lay out its parts."""

    def __init__(self, name: str, parse_config: Callable, build_spec: Callable):
        self.name = name
        self.parse_config = parse_config  # dict (config.json) → typed config
        self.build_spec = build_spec      # typed config → ModelSpec


def register_architecture(name: str, parse_config: Callable, build_spec: Callable, *, replace=False):
    return ARCHITECTURES.register(name, ArchitectureEntry(name, parse_config, build_spec), replace=replace)


def is_supported_architecture(name: str) -> bool:
    _ensure_builtin()
    return name in ARCHITECTURES


def get_architecture(name: str) -> ArchitectureEntry:
    _ensure_builtin()
    return ARCHITECTURES.get(name)


_builtin_loaded = False


def _ensure_builtin() -> None:
    """Import the modules that register the built-in architecture and parts."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from . import parts  # noqa: F401  (registers part kinds)
    from .models import qwen2  # noqa: F401  (registers the architecture)
