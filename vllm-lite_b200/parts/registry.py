"""Registries from a description's `kind` to the class that implements it.

Seven families: mixers, feed-forwards, norms, position encodings, blocks, embeddings and
output heads.
A class of any family offers

    declare(spec) -> {relative tensor name: TensorDecl}      (static, CPU only)
    __init__(spec, weights, ctx)                              (binds tensors)

and the family's own forward (see `parts.base`).  Mixers also offer
`cache_need(spec)` (static, CPU only), which says what they keep per request.
A new part is added by registering its class under a new kind; nothing in the
framework lists the kinds.
"""
from __future__ import annotations


class PartRegistry:
    def __init__(self, family: str):
        self.family = family
        self._classes = {}

    def register(self, kind: str, cls=None, *, replace: bool = False):
        def put(c):
            if kind in self._classes and not replace and self._classes[kind] is not c:
                raise KeyError(f"{self.family} kind {kind!r} is already registered")
            self._classes[kind] = c
            return c
        return put if cls is None else put(cls)

    def unregister(self, kind: str):
        self._classes.pop(kind, None)

    def get(self, kind: str):
        try:
            return self._classes[kind]
        except KeyError:
            raise KeyError(f"no {self.family} registered under kind {kind!r}; "
                           f"registered: {', '.join(sorted(self._classes)) or '(none)'}") from None

    def kinds(self):
        return sorted(self._classes)


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITIONS = PartRegistry("position encoding")
BLOCKS = PartRegistry("block")
EMBEDDINGS = PartRegistry("embedding")
HEADS = PartRegistry("output head")
