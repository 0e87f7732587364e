"""The one step function: a batch of (request, its next tokens) goes through the model as
one flat batch, from the cache that earlier steps left, and logits come back at the wanted
places only.

An entry may be a whole prompt, any portion of one (down to a single token), or one decoded
token; entries of all kinds share a step.  The reference has five cached forward entry
points, each for one batch shape, and none takes part of a prompt or mixes prompts with
decode rows (src/model/model.cpp:1091-1135, 1211-1314, 1316-1354, 1356-1446, 1448-1572);
its one packed [3, A] host-to-device transfer per step (model.cpp:1522-1538) is kept as
one pinned metadata buffer per step here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext
from ..parts.build import Model


class StepError(RuntimeError):
    pass


class OutOfPages(StepError):
    """A step needs more pages than the pool has free; nothing was run."""


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are asked for


def device_error_text(code: int) -> str:
    """What a non-zero device error flag means."""
    if code >= 10:
        return f"a bounded wait inside a tensor-memory kernel ran out (code {code}); the step's results are not valid"
    return f"a kernel met a token without a valid page (code {code}): the block table and the request's length disagree"


class Engine:
    """A model, its cache, and step().  Owns no policy: who runs when is the scheduler's."""

    def __init__(self, model: Model, cache: CacheManager):
        if not model.bound:
            raise StepError("the model has no weights bound")
        self.model, self.cache = model, cache
        self.device = model.rt.device
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.tokens_run = 0
        self.max_step_tokens: Optional[int] = None      # set when the cache's window groups were sized on this promise
        self._pinned: List[Optional[torch.Tensor]] = [None] * 4     # ring of staging buffers
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._pinned_next = 0

    @property
    def parameter_count(self) -> int:
        """Elements of every tensor the model declares (a tied head counts once)."""
        total = 0
        for spec in self.model.expected_tensors().values():
            n = 1
            for s in spec.shape:
                n *= int(s)
            total += n
        return total

    # ------------------------------------------------------------------ batch assembly
    def _pinned_buffer(self, n: int):
        """A pinned staging buffer that no copy in flight still reads."""
        i = self._pinned_next
        self._pinned_next = (i + 1) % len(self._pinned)
        if self._pinned_events[i] is not None:
            self._pinned_events[i].synchronize()
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            size = max(1024, 1 << (n - 1).bit_length())
            self._pinned[i] = torch.empty(size, dtype=torch.int32, pin_memory=True)
        return i, self._pinned[i]

    def build_context(self, entries: Sequence[StepEntry], patch=None) -> StepContext:
        """`patch` = (tokens of an earlier step on the device [int32], [(place among this step's flat tokens, index
        into that tensor), ...]): input tokens the host does not know yet because the step that selects them has
        not been read back.  The host packs a stand-in (token 0) and a small kernel, queued behind the metadata's
        upload, puts the selected tokens in their places before the embedding reads them."""
        spec, cache = self.model.spec, self.cache
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        pos0, counts = [], []
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not cache.has(e.request):
                raise StepError(f"request {e.request!r} is not live in the cache")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            if self.max_step_tokens and n > self.max_step_tokens:
                raise StepError(f"request {e.request!r} brings {n} tokens in one step; the cache was sized for at most "
                                f"{self.max_step_tokens}")
            p = cache.length(e.request)
            if p + n > spec.max_position:
                raise StepError(f"request {e.request!r} would hold {p + n} tokens, beyond max_position "
                                f"{spec.max_position}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.request!r} wants logits at place {w} of {n} tokens")
            pos0.append(p)
            counts.append(n)
        A, T = len(entries), sum(counts)
        R = sum(len(e.want) for e in entries)
        # pages for every entry, or none of the step runs
        for e, p, n in zip(entries, pos0, counts):
            if not cache.reserve(e.request, p + n):
                raise OutOfPages(f"no pages left for request {e.request!r} to grow from {p} to {p + n} tokens")
        groups = list(cache.groups)
        requests = [e.request for e in entries]
        tables = {g: cache.block_table(g, requests) for g in groups}
        widths = {g: len(tables[g][0]) for g in groups}

        pairs = list(patch[1]) if patch is not None else []
        P = len(pairs)
        for place, _ in pairs:
            if not 0 <= place < T:
                raise StepError(f"a token patch names place {place} of {T} tokens")
        total = 3 * T + (A + 1) + 3 * A + R + sum(A * w for w in widths.values()) + 2 * P
        ring_index, host = self._pinned_buffer(total)
        arr = host.numpy()
        cursor = 0

        def take(n):
            nonlocal cursor
            view = (cursor, cursor + n)
            cursor += n
            return view

        s_tok, s_pos, s_seq = take(T), take(T), take(T)
        s_starts, s_pos0, s_lens, s_slots, s_rows = take(A + 1), take(A), take(A), take(A), take(R)
        s_tables = {g: take(A * widths[g]) for g in groups}
        s_patch_to, s_patch_from = take(P), take(P)

        tok = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tok.min() < 0 or tok.max() >= spec.vocab_size:
            raise StepError(f"token id outside the vocabulary [0, {spec.vocab_size})")
        starts = np.zeros(A + 1, dtype=np.int32)
        starts[1:] = np.cumsum(counts)
        arr[s_tok[0]:s_tok[1]] = tok
        arr[s_pos[0]:s_pos[1]] = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, counts)])
        arr[s_seq[0]:s_seq[1]] = np.repeat(np.arange(A, dtype=np.int32), counts)
        arr[s_starts[0]:s_starts[1]] = starts
        arr[s_pos0[0]:s_pos0[1]] = pos0
        arr[s_lens[0]:s_lens[1]] = np.asarray(pos0) + np.asarray(counts)
        slots_host = [cache.slot(q) for q in requests]
        arr[s_slots[0]:s_slots[1]] = slots_host
        rows = [int(starts[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
        arr[s_rows[0]:s_rows[1]] = rows
        for g in groups:
            arr[s_tables[g][0]:s_tables[g][1]] = np.asarray(tables[g], dtype=np.int32).reshape(-1)

        if P:
            arr[s_patch_to[0]:s_patch_to[1]] = [place for place, _ in pairs]
            arr[s_patch_from[0]:s_patch_from[1]] = [index for _, index in pairs]

        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(host[:total], non_blocking=True)               # the step's one metadata transfer
        if P:
            from ..kernels import ops
            ops.scatter_int(dev[s_tok[0]:s_tok[1]], dev[s_patch_to[0]:s_patch_to[1]], patch[0], dev[s_patch_from[0]:s_patch_from[1]])
        event = self._pinned_events[ring_index] or torch.cuda.Event()
        event.record()
        self._pinned_events[ring_index] = event

        def d(view):
            return dev[view[0]:view[1]]

        return StepContext(
            num_tokens=T, num_seqs=A, token_ids=d(s_tok), positions=d(s_pos), token_seq=d(s_seq),
            seq_starts=d(s_starts), seq_pos0=d(s_pos0), seq_lens=d(s_lens),
            block_tables={g: d(s_tables[g]).view(A, widths[g]) for g in groups},
            state_slots=d(s_slots), logit_rows=d(s_rows), error_flag=self.error_flag,
            seq_starts_host=[int(x) for x in starts], seq_pos0_host=list(pos0), state_slots_host=slots_host,
            max_new_tokens=max(counts), max_seq_len=max(p + n for p, n in zip(pos0, counts)))

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], tensor_sink=None, patch=None) -> torch.Tensor:
        """Run the given tokens; returns fp32 logits [wanted, vocab] on the device, in the order
        of the entries and of each entry's `want`.  Lengths advance only if the step ran.
        `tensor_sink(name, tensor)`: receives the step's intermediate tensors (a tensor trace; see
        StepContext.tensor_sink).  `patch`: see build_context."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        ctx = self.build_context(entries, patch)
        ctx.tensor_sink = tensor_sink
        views = self.cache_views(ctx)
        logits = self.model.forward(ctx, views)
        for e, p in zip(entries, ctx.seq_pos0_host):
            self.cache.commit(e.request, p + len(e.tokens))
        self.steps_run += 1
        self.tokens_run += ctx.num_tokens
        return logits

    def cache_views(self, ctx: StepContext) -> Dict[str, object]:
        cache = self.cache
        views = {}
        for name in self.model.cache_entries:
            group = cache.entry_group.get(name)
            views[name] = cache.view(name, ctx.block_tables[group] if group is not None else None,
                                     ctx.state_slots, ctx.state_slots_host)
        return views

    def check_device_errors(self) -> None:
        """Kernels raise a flag instead of touching memory outside the pool; reading it costs a
        synchronisation, so callers do it where they synchronise anyway."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise StepError(device_error_text(code))
        self.cache.check_guards()              # nothing to read unless the cache was made with guard pages
