"""From a `ModelSpec` to a runnable model: build every part, collect the tensors they
expect under their full names, bind them once loaded, and run the execution list.

The reference's counterpart is `TransformerModel::Impl` (src/model/model.cpp:912-941:
embedding, vector of blocks, final norm, optional head) with the forward loop of
:1043-1087; here the loop walks `spec.order`, which may name a layer twice or let a run
read an earlier run's cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Part, Runtime,
                   StepContext, WeightSpec, make)


@dataclass
class CacheEntry:
    """One cache that some run owns: its name and what its mixer needs."""
    name: str
    need: object                  # PagedKVNeed | FixedStateNeed


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        self.embedding = make(EMBEDDINGS, "embedding", spec.embedding, rt)
        self.position = make(POSITION_ENCODINGS, "position encoding", spec.position, rt)
        self.final_norm = make(NORMS, "norm", spec.final_norm, rt)
        self.head = make(HEADS, "head", spec.head, rt)
        self.blocks = []
        self._parts: List[Tuple[str, Part]] = [("", self.embedding), (spec.position.params.get("prefix", ""), self.position),
                                               (spec.final_norm.params.get("prefix", ""), self.final_norm),
                                               ("", self.head)]
        for layer in spec.layers:
            position = self.position
            if "position" in layer.mixer.params:                 # a layer may bring its own encoding
                position = make(POSITION_ENCODINGS, "position encoding", layer.mixer.params["position"], rt)
                self._parts.append((layer.prefix + layer.mixer.params["position"].params.get("prefix", ""), position))
            mixer_cls = MIXERS.get(layer.mixer.kind)
            if mixer_cls is None:
                raise KeyError(f"unknown mixer kind {layer.mixer.kind!r}; registered: {', '.join(sorted(MIXERS))}")
            mixer = mixer_cls(layer.mixer.params, rt, position)
            feed_forward = make(FEED_FORWARDS, "feed-forward", layer.feed_forward, rt)
            mixer_norm = make(NORMS, "norm", layer.mixer_norm, rt)
            ffn_norm = make(NORMS, "norm", layer.ffn_norm, rt)
            block = make(BLOCKS, "block", layer.block, rt, mixer_norm, mixer, ffn_norm, feed_forward)
            self.blocks.append(block)
            for part, ps in ((mixer_norm, layer.mixer_norm), (mixer, layer.mixer), (ffn_norm, layer.ffn_norm),
                             (feed_forward, layer.feed_forward)):
                self._parts.append((layer.prefix + ps.params.get("prefix", ""), part))
        # caches: one entry per owning run
        self.cache_entries: Dict[str, CacheEntry] = {}
        self.run_cache: List[Tuple[Optional[str], bool]] = []    # per run: (cache name, owns it)
        for i, run in enumerate(spec.order):
            need = self.blocks[run.layer].mixer.cache_need()
            if need is None:
                self.run_cache.append((None, False))
                continue
            name = spec.cache_name(i)
            owns = run.read_cache_of is None
            if owns:
                if name in self.cache_entries:
                    raise ValueError(f"two runs own the cache {name!r}")
                self.cache_entries[name] = CacheEntry(name, need)
            else:
                if name not in self.cache_entries:
                    raise ValueError(f"order[{i}] reads cache {name!r}, which no earlier run owns")
                if type(self.cache_entries[name].need) is not type(need):
                    raise ValueError(f"order[{i}] reads cache {name!r} of another kind than its mixer needs")
            self.run_cache.append((name, owns))
        self.bound = False

    def parts(self) -> List[Part]:
        """Every part of the model, each once."""
        seen, out = set(), []
        for _, part in self._parts:
            if id(part) not in seen:
                seen.add(id(part))
                out.append(part)
        return out

    # --- weights ----------------------------------------------------------------------
    def expected_tensors(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for prefix, part in self._parts:
            for local, ws in part.weight_specs().items():
                full = prefix + local
                if full in out and out[full] != ws:
                    raise ValueError(f"tensor {full!r} is declared twice with different specs")
                out[full] = ws
        return out

    def tolerated_extra_tensors(self) -> List[str]:
        """Names a checkpoint may carry although no part wants them: a redundant head matrix
        when the head is tied to the embedding table."""
        params = self.spec.head.params
        return [params["name"]] if params.get("tied_to") is not None and "name" in params else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """`tensors`: full name -> device tensor, already in the dtype policy of the runtime."""
        for prefix, part in self._parts:
            local = {name: tensors[prefix + name] for name in part.weight_specs()}
            tied = getattr(part, "tied_to", None)
            if tied is not None:
                local[tied] = tensors[tied]
            part.bind(local)
        self.bound = True

    # --- forward ------------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: Dict[str, object]) -> torch.Tensor:
        """Run the tokens of `ctx` through the execution list; returns fp32 logits [R, V] at
        ctx.logit_rows.  `caches`: cache name -> writable view for this step."""
        if not self.bound:
            raise RuntimeError("model weights are not bound")
        ctx.step_values.clear()              # nothing computed from an earlier step's positions or tokens survives
        residual = self.embedding.forward(ctx.token_ids)
        self.position.on_embedding(residual, ctx)
        delta = None
        for i, run in enumerate(self.spec.order):
            name, owns = self.run_cache[i]
            view = None
            if name is not None:
                view = caches[name]
                if not owns:
                    view = _read_only(view)
            residual, delta = self.blocks[run.layer].forward(residual, delta, ctx, view)
        R = ctx.logit_rows.shape[0]
        if R == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        if delta is not None:
            from ..kernels import ops
            ops.add_inplace(residual, delta)
        rows = torch.empty((R, self.spec.hidden_size), dtype=self.rt.dtype, device=residual.device)
        self.final_norm.forward(residual, rows, rows=ctx.logit_rows)
        return self.head.forward(rows, ctx.error_flag)


def _read_only(view):
    import copy
    v = copy.copy(view)
    v.writable = False
    return v


def build_model(spec: ModelSpec, rt: Runtime) -> Model:
    return Model(spec, rt)
