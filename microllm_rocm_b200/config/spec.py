"""Architecture-neutral description of a decoder: which parts make up each layer,
and in which order the layers run.

A `ModelSpec` is pure data.  An architecture (see `registry.py`) turns its own typed
configuration into one; the builder in `parts/build.py` turns the spec into parts.
Nothing in here knows a model family: sizes and constants travel as parameters of
`PartSpec`, and every layer names its own mixer, feed-forward and norms, so one model
may mix different kinds layer by layer.

The run order is data too.  `ModelSpec.order` is a list of `RunSpec`; the same layer
may appear twice (its weights are shared, each occurrence gets a cache of its own
unless told otherwise), and a run may read the cache that an earlier run wrote
(`read_cache_of`), in which case it stores nothing itself.

The reference hard-wires one block class with one attention and one feed-forward
(src/model/model.cpp:820-908) and a fixed loop over `blocks` (model.cpp:1043-1068);
this module is what replaces that wiring.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by `kind` (a registry key) with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):  # params is a dict; hash on a stable rendering
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward.

    `prefix` is the layer's tensor-name prefix in the weight file; each part appends
    its own sub-prefix (given in its PartSpec params as ``prefix``).
    """
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class RunSpec:
    """One entry of the execution list.

    layer          index into `ModelSpec.layers`
    cache          name of the cache entry this run owns (None: derived from its
                   place in the list, so a layer that runs twice gets two caches)
    read_cache_of  index into `ModelSpec.order` of an EARLIER run whose cache this
                   run reads instead of writing one of its own
    """
    layer: int
    cache: Optional[str] = None
    read_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    position: PartSpec
    layers: List[LayerSpec]
    order: List[RunSpec]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_position <= 0:
            raise ValueError("hidden_size, vocab_size and max_position must be positive")
        if not self.layers or not self.order:
            raise ValueError("a model needs at least one layer and one run")
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, which does not exist")
            if run.read_cache_of is not None:
                if not 0 <= run.read_cache_of < i:
                    raise ValueError(
                        f"order[{i}] may only read the cache of an earlier run, "
                        f"not {run.read_cache_of}")
                if self.order[run.read_cache_of].read_cache_of is not None:
                    raise ValueError(
                        f"order[{i}] reads the cache of run {run.read_cache_of}, "
                        "which owns none")

    def cache_name(self, run_index: int) -> str:
        """Name of the cache entry that run `run_index` reads and (if owner) writes."""
        run = self.order[run_index]
        if run.read_cache_of is not None:
            return self.cache_name(run.read_cache_of)
        return run.cache if run.cache is not None else f"run{run_index}"
