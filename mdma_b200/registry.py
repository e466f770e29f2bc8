"""Name -> factory registries.

One registry maps an architecture name (config.json `architectures[0]` or
`model_type`) to its configuration class and model description; four more map
the kinds of parts (mixer, feed-forward, norm, position encoding, block
arrangement) to their classes.  Unknown names are rejected with the list of
registered ones; nothing is approximated (the reference's rule for unknown
`general.architecture`, src/model.rs:157-168, src/model/preflight.rs:31-43).
"""
from __future__ import annotations

from typing import Generic, Iterator, TypeVar

T = TypeVar("T")


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message otherwise
        return self.args[0] if self.args else ""


class Registry(Generic[T]):
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, T] = {}

    def register(self, name: str, item: T = None, *, replace: bool = False):
        """Register `item` under `name`; usable as a decorator when `item` is omitted."""
        def put(obj: T) -> T:
            if name in self._items and not replace:
                raise RegistryError(f"{self.what} {name!r} is already registered")
            self._items[name] = obj
            return obj
        if item is None:
            return put
        return put(item)

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> T:
        try:
            return self._items[name]
        except KeyError:
            raise RegistryError(
                f"unknown {self.what} {name!r}; registered: {sorted(self._items)}") from None

    def __contains__(self, name: str) -> bool:
        return name in self._items

    def __iter__(self) -> Iterator[str]:
        return iter(sorted(self._items))


ARCHITECTURES: Registry = Registry("architecture")
MIXERS: Registry = Registry("mixer")
FEED_FORWARDS: Registry = Registry("feed-forward")
NORMS: Registry = Registry("norm")
POSITIONS: Registry = Registry("position encoding")
BLOCKS: Registry = Registry("block arrangement")
EMBEDDINGS: Registry = Registry("embedding")
HEADS: Registry = Registry("output head")
