"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from a `PartSpec`'s params and a `Runtime` (device + compute dtype).  It
declares the tensors it wants by LOCAL name (`weight_specs`), receives them already on the
device and in the engine's dtype policy (`bind`), and then computes.  No part knows which
model it sits in, which layer it is, or what runs before and after it.

Kinds (each has a registry; `register_*` adds to it, tests may add their own):

  Norm             forward(x[T,H] f32, out)            and add_forward(residual, delta, out)
  PositionEncoding rotary_table() for mixers that rotate q/k, on_embedding() for additive ones
  Mixer            cache_need(); forward(x[T,H], ctx, cache_view) -> delta[T,H] f32
  FeedForward      forward(x[T,H], ctx) -> delta[T,H] f32
                   (a delta may also be [S,T,H]: partial sums that the next norm adds up)
  Block            the arrangement of norm/mixer/feed-forward around the residual stream

`StepContext` is everything a part may know about the batch it is running: flat tokens with
their absolute positions and the index of their sequence, per-sequence extents, and the
per-group block tables and state slots of the cache manager.

The reference welds these together in one file: Linear/Norm/Attention/FeedForward/Block
are private classes of the one model (src/model/model.cpp:280-908).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


# ----------------------------------------------------------------------------- runtime
@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype                      # torch.float32 (true 32-bit path) or torch.bfloat16

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


# ----------------------------------------------------------------------------- weights
@dataclass(frozen=True)
class WeightSpec:
    """What a part expects of one tensor.

    role   'matrix' / 'table': kept in the compute dtype (bf16 or f32)
           'vector': norm weights, biases; always f32 on the device (their math is f32)
           'int_table': integer tables, int32 on the device
    init   how the random-weights mode draws it: ('normal', std) or ('one_plus_normal', std)
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[str, float] = ("normal", 0.02)


# ----------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values that grow with the tokens.  `window`: only the last `window` keys are
    ever read (pages behind it may be given back while the request lives); None: all keys.
    `dtype`: what the pages store; None: the runtime's compute dtype."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class FixedStateNeed:
    """Per-request state of a fixed size, whatever the number of tokens."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PagedKVView:
    pages: torch.Tensor            # [num_pages, 2, NKV, page_size, D]
    block_table: torch.Tensor      # [A, max_blocks] int32, this step's sequences, this group
    page_size: int
    writable: bool                 # False: the run reads a cache another run wrote


@dataclass
class StateView:
    storage: torch.Tensor          # [num_slots, *shape]
    slots: torch.Tensor            # [A] int32 slot of each sequence of the step
    slots_host: List[int]
    writable: bool


# ----------------------------------------------------------------------------- step context
@dataclass
class StepContext:
    """One step's batch as the parts see it.  Device tensors are int32."""
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T] absolute position of each token in its sequence
    token_seq: torch.Tensor        # [T] which sequence (0..A-1) the token belongs to
    seq_starts: torch.Tensor       # [A+1] first flat index of each sequence's tokens
    seq_pos0: torch.Tensor         # [A] tokens the sequence held before this step
    seq_lens: torch.Tensor         # [A] tokens it holds after this step
    block_tables: Dict[str, torch.Tensor]   # cache group -> [A, max_blocks]
    state_slots: torch.Tensor      # [A]
    logit_rows: torch.Tensor       # [R] flat token indices whose logits are wanted
    error_flag: torch.Tensor       # [1] int32, kernels raise it on a bad page or slot
    # host mirrors, for parts that plan launches on the host
    seq_starts_host: List[int] = field(default_factory=list)
    seq_pos0_host: List[int] = field(default_factory=list)
    state_slots_host: List[int] = field(default_factory=list)
    max_new_tokens: int = 0        # longest run of new tokens of one sequence
    max_seq_len: int = 0           # longest sequence after the step
    extras: Dict[str, Any] = field(default_factory=dict)   # scratch buffers and launch plans shared by parts
    # results computed from the step's device state (a table of this step's angles, say): valid for ONE forward;
    # the model empties it before every forward, also when the context itself lives on (a captured decode step)
    step_values: Dict[Any, Any] = field(default_factory=dict)
    # When set, the model hands it (name, tensor) after the embedding, after every run of the execution list
    # (residual stream and the delta not yet added to it), after the final norm and for the logits: a per-step
    # tensor trace.  Such a step runs every layer call by call.
    tensor_sink: Optional[Callable[[str, torch.Tensor], None]] = None

    @property
    def decode_only(self) -> bool:
        return self.max_new_tokens == 1

    def buffer(self, role: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Scratch of this step for one role ("attention.q", "block.normed", ...): the same tensor every time
        the role, shape and dtype come back, so the layers of a model share it (each is done with it before the
        next one writes) and a step costs one allocation per role instead of one per layer.  A part names its
        roles after itself, and may only ask for a buffer whose content nobody reads after the part has returned
        and the next part has consumed what it returned."""
        key = (role, shape, dtype)
        t = self.extras.get(key)
        if t is None:
            t = self.extras[key] = torch.empty(shape, dtype=dtype, device=self.token_ids.device)
        return t


def scratch(ctx: Optional[StepContext], role: str, shape: Tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
    """ctx.buffer(...), or a fresh tensor for a part that is run without a step around it."""
    if ctx is None:
        return torch.empty(shape, dtype=dtype, device=device)
    return ctx.buffer(role, shape, dtype)


# ----------------------------------------------------------------------------- part kinds
class Part:
    """Common surface: declare tensors, receive them."""
    prefix: str = ""

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def fused_tensors(self) -> Dict[str, Tuple[WeightSpec, List[Tuple[str, int]]]]:
        """Tensors this part keeps FUSED on the device although the checkpoint stores their pieces apart:
        local name of the fused tensor -> (its spec, [(local name of a piece, first row it occupies), ...]).
        The loader then allocates the fused tensor once and streams each piece straight into its rows, and
        `bind` receives the fused tensor under its local name instead of the pieces.  Default: nothing is fused
        (a part may still join pieces in `bind`, at the price of holding them twice for a moment)."""
        return {}

    def kernel_sources(self) -> List[Tuple[str, dict]]:
        """(source file, defines) of the kernel objects this part will ask for beyond those every model needs,
        so that they are compiled together, in parallel, before the first step instead of one by one inside it."""
        return []

    # Layers of equal structure issue the same launches; only their own tensors differ.  A part that says so lets
    # the model record one layer's launches and issue them again, natively, for the others (kernels/replay.py).
    def replay_key(self):
        """A hashable description of everything but the part's own tensors that decides which launches its
        forward makes and with which arguments (sizes, constants, options), or None: this part's forward does
        work that a recording of launcher calls would miss (tensor-framework operations, host-side state), so
        its layers always run call by call.  Default: None."""
        return None

    def own_tensors(self) -> List[Optional[torch.Tensor]]:
        """The device tensors this part owns, in a fixed order (None for an absent optional one): what differs
        between two parts with the same replay_key."""
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor, out: torch.Tensor) -> None:
        """residual += delta in place, then out = norm(residual)."""
        raise NotImplementedError


@dataclass(frozen=True)
class RotaryTable:
    inv_freq: torch.Tensor         # [rotary_dim/2] f32 on the device
    rotary_dim: int
    interleaved: bool


class PositionEncoding(Part):
    def rotary_table(self, head_dim: int) -> Optional[RotaryTable]:
        """Inverse frequencies for mixers that rotate q and k; None if this encoding does
        nothing there."""
        return None

    def on_embedding(self, x: torch.Tensor, ctx: StepContext) -> None:
        """Hook for encodings that add to the embedded tokens (in place); default none."""
        return None


class Mixer(Part):
    # True when forward() only launches work on the current stream from device-resident
    # inputs (no host mirrors of the context, no synchronisation): such a mixer may be
    # captured into a CUDA graph for steady decoding.
    graph_safe = False

    def cache_need(self):
        """PagedKVNeed, FixedStateNeed or None."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError

    # A mixer may plan its launches on the host from the lengths of the step's sequences and keep the plan in
    # ctx.extras; a captured decode step freezes that plan while the sequences grow.  The two hooks let whoever
    # holds such a context ask whether the plan still suits, and drop it, without knowing what the plan is.
    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        """Whether launches planned in `ctx` would be cut differently once the longest sequence holds
        `max_seq_len` tokens.  Default: the mixer plans nothing that depends on lengths."""
        return False

    def forget_plans(self, ctx: StepContext) -> None:
        """Drop this mixer's plans from `ctx`; the next forward plans anew."""
        return None

    def plan_group(self):
        """Mixers with equal plan_group share their plans in a context (the layers of a model, usually): asking one
        of them whether the plans are stale answers for all.  Default: every mixer plans for itself."""
        return id(self)


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of two norms, a mixer and a feed-forward around the residual stream.
    `forward` gets the residual and a delta not yet added to it (or None) and returns the
    same pair, so the add can be fused into whichever norm comes next."""

    def __init__(self, params, rt, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, feed_forward: FeedForward):
        raise NotImplementedError

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache):
        raise NotImplementedError

    def replay_key(self):
        """As Part.replay_key, for the whole block; in addition the block promises that with equal keys its
        forward returns the same (residual, delta) tensors for every layer of a step (scratch by role from
        ctx.buffer, never a fresh tensor).  Default: None."""
        return None

    def own_tensors(self) -> List[Optional[torch.Tensor]]:
        return []


# ----------------------------------------------------------------------------- registries
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}
EMBEDDINGS: Dict[str, Callable] = {}
HEADS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], what: str):
    def deco_factory(kind: str, *, replace: bool = False):
        def deco(cls):
            if kind in table and not replace:
                raise KeyError(f"{what} {kind!r} is already registered")
            table[kind] = cls
            return cls
        return deco
    return deco_factory


register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_block = _register(BLOCKS, "block")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def make(table: Dict[str, Callable], what: str, spec, *args, **kwargs):
    if spec.kind not in table:
        raise KeyError(f"unknown {what} kind {spec.kind!r}; registered: {', '.join(sorted(table))}")
    return table[spec.kind](spec.params, *args, **kwargs)
