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
        # Layers of equal structure are recorded once per step and issued again natively (kernels/replay.py);
        # False runs every layer call by call.
        self.replay_layers = True
        self.layers_replayed = 0             # runs issued from a recording so far
        self._replay_keys: Optional[List[object]] = None

    def parts(self) -> List[Part]:
        """Every part of the model, each once."""
        seen, out = set(), []
        for _, part in self._parts:
            if id(part) not in seen:
                seen.add(id(part))
                out.append(part)
        return out

    # --- layers of equal structure --------------------------------------------------------
    def _layer_replay_keys(self) -> List[object]:
        """Per run of the execution list: what decides its launches besides its own tensors, or None."""
        if self._replay_keys is None:
            keys = []
            for i, run in enumerate(self.spec.order):
                key = self.blocks[run.layer].replay_key()
                name, owns = self.run_cache[i]
                group = None
                if name is not None:
                    need = self.cache_entries[name].need
                    group = (type(need).__name__, getattr(need, "window", None), getattr(need, "dtype", None))
                keys.append(None if key is None else (key, owns, group))
            self._replay_keys = keys
        return self._replay_keys

    @staticmethod
    def _run_pointers(block, view) -> List[int]:
        return [0 if t is None else t.data_ptr() for t in list(block.own_tensors()) + _view_tensors(view)]

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

    def placements(self):
        """Where each checkpoint tensor goes on the device.  Returns (destinations, pieces):
        destinations: full name of a device tensor -> its WeightSpec (a fused tensor, or the checkpoint tensor itself);
        pieces: full checkpoint name -> (full destination name, first row)."""
        destinations: Dict[str, WeightSpec] = {}
        pieces: Dict[str, Tuple[str, int]] = {}
        for prefix, part in self._parts:
            fused = part.fused_tensors()
            inside = {}
            for dest, (spec, parts_of) in fused.items():
                destinations[prefix + dest] = spec
                for local, row in parts_of:
                    inside[local] = (prefix + dest, row)
            for local, ws in part.weight_specs().items():
                if local in inside:
                    pieces[prefix + local] = inside[local]
                else:
                    destinations.setdefault(prefix + local, ws)
                    pieces[prefix + local] = (prefix + local, 0)
        return destinations, pieces

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """`tensors`: full name -> device tensor, already in the dtype policy of the runtime; either under the
        checkpoint's names or under the destination names of `placements()`."""
        for prefix, part in self._parts:
            fused = part.fused_tensors()
            if fused and all(prefix + dest in tensors for dest in fused):
                covered = {local for _, parts_of in fused.values() for local, _ in parts_of}
                local = {dest: tensors[prefix + dest] for dest in fused}
                local.update({name: tensors[prefix + name] for name in part.weight_specs() if name not in covered})
                tied = getattr(part, "tied_to", None)
                if tied is not None:
                    local[tied] = tensors[tied]
                part.bind(local)
                continue
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
        sink = ctx.tensor_sink
        if sink is not None:
            sink("embedding", residual)
        keys = self._layer_replay_keys() if self.replay_layers and sink is None else None
        recordings = {}                      # structure of a run -> (recording, the recorded run's own pointers) | None
        for i, run in enumerate(self.spec.order):
            name, owns = self.run_cache[i]
            view = None
            if name is not None:
                view = caches[name]
                if not owns:
                    view = _read_only(view)
            block = self.blocks[run.layer]
            key = keys[i] if keys is not None and i > 0 and delta is not None else None
            if key is None:
                # the first run of a step plans launches and makes the step's tables: it always runs call by call
                residual, delta = block.forward(residual, delta, ctx, view)
                if sink is not None:
                    sink(f"run{i}.layer{run.layer}.residual", residual)
                    sink(f"run{i}.layer{run.layer}.delta", delta)
                continue
            pointers = self._run_pointers(block, view)
            if key not in recordings:
                from ..kernels.replay import Recorder, Recording
                with Recorder() as recorder:
                    out_residual, out_delta = block.forward(residual, delta, ctx, view)
                recording = None
                if (out_residual is residual and out_delta is not None and delta is not None
                        and out_delta.data_ptr() == delta.data_ptr() and recorder.unrecordable is None):
                    recording = Recording(recorder)
                    if not _swappable(recording, block, view):
                        recording = None
                recordings[key] = (recording, pointers) if recording is not None else None
                residual, delta = out_residual, out_delta
                continue
            entry = recordings[key]
            if entry is None:
                residual, delta = block.forward(residual, delta, ctx, view)
                continue
            recording, base = entry
            recording.replay(list(zip(base, pointers)))
            self.layers_replayed += 1
        R = ctx.logit_rows.shape[0]
        if R == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        if delta is not None:
            from ..kernels import ops
            ops.add_inplace(residual, delta)
        rows = torch.empty((R, self.spec.hidden_size), dtype=self.rt.dtype, device=residual.device)
        self.final_norm.forward(residual, rows, rows=ctx.logit_rows)
        logits = self.head.forward(rows, ctx.error_flag)
        if sink is not None:
            sink("final_norm", rows)
            sink("logits", logits)
        return logits


def _view_tensors(view) -> List[Optional[torch.Tensor]]:
    if view is None:
        return []
    return [getattr(view, "pages", None), getattr(view, "storage", None)]


def _swappable(recording, block, view) -> bool:
    """Every pointer a recorded launch takes into a tensor the layer owns must be that tensor's base address:
    only those can be replaced by another layer's tensor.  (A launcher handed `weight + offset` would keep
    reading the recorded layer's weight.)"""
    owned = [t for t in list(block.own_tensors()) + _view_tensors(view) if t is not None]
    ranges = [(t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()) for t in owned]
    for p in recording.pointers:
        for lo, hi in ranges:
            if lo < p < hi:
                return False
    return True


def _read_only(view):
    import copy
    v = copy.copy(view)
    v.writable = False
    return v


def build_model(spec: ModelSpec, rt: Runtime) -> Model:
    return Model(spec, rt)
