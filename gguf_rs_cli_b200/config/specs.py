"""Architecture-neutral description of a decoder: which parts make each layer, with
which constants and which tensors, and in which order the layers run.

An architecture's builder turns its typed configuration into a `ModelSpec`; the
generic decoder (`models/decoder.py`) builds parts from the registries in
`parts/registry.py` and never looks at the architecture's name again.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: `kind` names a class in a part registry, `params` are its
    sizes and constants, `tensors` maps the part's local tensor names to the names
    in the model folder."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)

    def key(self) -> str:
        """Stable text of kind and constants: equal keys may share tables."""
        return self.kind + repr(sorted((k, repr(v)) for k, v in self.params.items()))


@dataclass(frozen=True)
class LayerSpec:
    """A block and its parts.  `block` names the arrangement (how norms, mixer and
    feed-forward are wired around the residual stream)."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class Run:
    """One entry of the run order: layer `layer` runs here.  `cache_of` is None when
    this run owns cache storage (if its mixer needs any), or the index of an earlier
    run whose keys and values this run reads instead of making its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[Run]
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    stop_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    # shell-style patterns of tensor names a folder may hold although no part asks for them
    ignored_tensors: List[str] = field(default_factory=list)

    def validate(self) -> None:
        for r, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{r}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < r:
                    raise ValueError(f"schedule[{r}].cache_of={run.cache_of} must name an earlier run")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{r}].cache_of={run.cache_of} names a run that owns no cache")
