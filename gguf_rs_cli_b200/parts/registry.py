"""Registries of the parts a layer is made of.  A `PartSpec.kind` names a class in
the registry of its role; the decoder builds layers from these and knows no part by
name.  A new part is a class with the role's interface (see `base.py`) and one
`register_*` call; nothing else in the package changes.
"""
from __future__ import annotations

from typing import Callable, Dict


class Registry:
    def __init__(self, role: str):
        self.role = role
        self._classes: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls: type) -> type:
            self._classes[kind] = cls
            return cls
        return deco

    def get(self, kind: str) -> type:
        if kind not in self._classes:
            raise KeyError(f"no {self.role} of kind {kind!r} is registered; known: {sorted(self._classes)}")
        return self._classes[kind]

    def kinds(self):
        return sorted(self._classes)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
