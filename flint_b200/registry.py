"""Name -> class tables for everything a model is put together from.

One table per kind of part and one for whole architectures.  A part registers under
a short name (``"attention"``, ``"layernorm"``); an architecture registers under the
string found in ``config.json``'s ``architectures[0]``.  The reference keeps the
architecture table as an enum matched on the checkpoint's architecture key and
fails with the list of known names (crates/thuban_architectures/src/loader.rs:39-60).
Registration is open: a test or a user module can add a part or an architecture
without touching the package.
"""
from __future__ import annotations

from .errors import ConfigError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, object] = {}

    def register(self, name: str, item=None, *, replace: bool = False):
        """``REG.register("name", cls)`` or ``@REG.register("name")``."""
        def put(obj):
            if name in self._items and not replace and self._items[name] is not obj:
                raise ConfigError(f"{self.what} {name!r} is already registered")
            self._items[name] = obj
            return obj
        return put if item is None else put(item)

    def unregister(self, name: str):
        self._items.pop(name, None)

    def get(self, name: str):
        try:
            return self._items[name]
        except KeyError:
            known = ", ".join(sorted(self._items)) or "(none)"
            raise ConfigError(f"unknown {self.what} {name!r}; registered: {known}") from None

    def names(self):
        return sorted(self._items)

    def __contains__(self, name):
        return name in self._items


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
ARCHITECTURES = Registry("architecture")
