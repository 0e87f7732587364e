"""Steady decoding as one captured CUDA graph whose inputs live on the device.

When every request of a step brings exactly one token (its last selected one), the step's
launches are always the same ~10 per layer; issuing them one by one from Python costs more
than the kernels take.  A `DecodeGraph` holds the step's metadata in fixed device buffers,
captures model forward + token selection + bookkeeping once, and replays it: the selected
token is written where the next replay's embedding reads it, positions and lengths advance
on the device, and the host only (a) makes sure each request has a page for its next token
and refreshes the device block table when one was added, and (b) reads the selected tokens.

The reference keeps tokens on the device for greedy decoding in the same spirit
(src/inference/generator.cpp:108-126: argmax writes into a device history that is the next
step's input) but launches every kernel of every step from the host.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import RELEASED
from ..kernels import ops
from ..parts.base import StepContext
from ..sampling.config import GenerationConfig
from .step import Engine, StepError, device_error_text


def graph_capable(engine: Engine) -> bool:
    return all(getattr(b.mixer, "graph_safe", False) for b in engine.model.blocks)


def _round_up_pow2(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


class DecodeGraph:
    def __init__(self, engine: Engine, batch: int, table_widths: Dict[str, int], host_io: bool = False):
        # host_io: the captured step begins with the copy of the requests' input tokens out of pinned host memory
        # and ends with the copy of the selected tokens (and the error flag) into pinned host memory, so that a
        # step costs the host ONE launch between writing the tokens and waiting for the answers.  Without it the
        # tokens stay where the sampler left them and the caller copies what it wants (a device-only loop).
        self.engine, self.batch, self.host_io = engine, batch, bool(host_io)
        self.widths = dict(table_widths)
        dev = engine.device
        A = batch
        cursor = 0

        def take(n, align=1):
            nonlocal cursor
            cursor = -(-cursor // align) * align
            view = (cursor, cursor + n)
            cursor += n
            return view

        self._s = {name: take(A) for name in ("tokens", "positions", "token_seq", "seq_pos0", "seq_lens", "slots",
                                              "logit_rows", "temperature", "top_k", "grows")}
        self._s["seq_starts"] = take(A + 1)
        self._s["seed"] = take(2 * A, align=2)
        self._s["draw"] = take(2 * A, align=2)
        self._dynamic_end = cursor
        self._tables = {g: take(A * w) for g, w in self.widths.items()}
        self.total = cursor
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=dev)
        self.out_host = torch.zeros(A + 1, dtype=torch.int32, pin_memory=True)     # tokens, then the error flag
        self.out_dev = torch.zeros(A + 1, dtype=torch.int32, device=dev)           # gathered by the step's last kernel
        self._upload_pending = False
        self._token_views = None
        self._tables_version = -1
        d = lambda name: self.dev[self._s[name][0]:self._s[name][1]]
        self.temperature = d("temperature").view(torch.float32)
        self.top_k = d("top_k")
        self.grows = d("grows")
        self.active = 0                # rows that belong to requests; the others only fill the captured batch up
        self.seed = d("seed").view(torch.int64)
        self.draw = d("draw").view(torch.int64)
        self.ctx = StepContext(
            num_tokens=A, num_seqs=A, token_ids=d("tokens"), positions=d("positions"), token_seq=d("token_seq"),
            seq_starts=d("seq_starts"), seq_pos0=d("seq_pos0"), seq_lens=d("seq_lens"),
            block_tables={g: self.dev[v[0]:v[1]].view(A, self.widths[g]) for g, v in self._tables.items()},
            state_slots=d("slots"), logit_rows=d("logit_rows"), error_flag=engine.error_flag,
            seq_starts_host=list(range(A + 1)), seq_pos0_host=[], state_slots_host=[], max_new_tokens=1, max_seq_len=1)
        self.views = engine.cache_views(self.ctx)
        self._planners = list({b.mixer.plan_group(): b.mixer for b in engine.model.blocks}.values())    # one mixer per shared plan
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.requests: List[Hashable] = []
        self._table_state: Dict[str, List[tuple]] = {}
        self.replays = 0

    # ------------------------------------------------------------------ host -> device state
    def _h(self, name):
        a, b = self._s[name]
        return self.host.numpy()[a:b]

    def load(self, requests: Sequence[Hashable], tokens: Sequence[int], lengths: Sequence[int],
             configs: Sequence[GenerationConfig], draws: Sequence[int]) -> None:
        """Set the device state: request i feeds `tokens[i]` at position `lengths[i]`.  Fewer requests than the
        captured batch: the remaining rows feed token 0 at position 0 of a sequence of their own that lives in the
        cache's spare page and slot and never grows; what they select is not read."""
        A = self.batch
        n = len(requests)
        if not 0 < n <= A:
            raise StepError("a decode graph serves at most the batch size it was built for")
        self._wait_upload()
        cache = self.engine.cache
        self.requests = list(requests)
        self.active = n
        pad = A - n
        self._h("tokens")[:] = list(tokens) + [0] * pad
        self._h("positions")[:] = list(lengths) + [0] * pad
        self._h("token_seq")[:] = np.arange(A)
        self._h("seq_pos0")[:] = list(lengths) + [0] * pad
        self._h("seq_lens")[:] = [x + 1 for x in lengths] + [1] * pad
        self._h("slots")[:] = [cache.slot(q) for q in requests] + [cache.pad_slot] * pad
        self._h("logit_rows")[:] = np.arange(A)
        self._h("seq_starts")[:] = np.arange(A + 1)
        self._h("grows")[:] = [1] * n + [0] * pad
        self._h("temperature").view(np.float32)[:] = [0.0 if c.greedy else c.temperature for c in configs] + [0.0] * pad
        self._h("top_k")[:] = [c.top_k for c in configs] + [0] * pad
        self._h("seed").view(np.int64)[:] = [c.seed for c in configs] + [0] * pad
        self._h("draw").view(np.int64)[:] = list(draws) + [0] * pad
        self._table_state = {}
        self._fill_tables()
        self._tables_version = cache.tables_version
        self.dev.copy_(self.host, non_blocking=True)
        self._mark_upload()
        self.ctx.max_seq_len = max(lengths) + 1

    def _mark_upload(self) -> None:
        self._upload_pending = True

    def _wait_upload(self) -> None:
        """The staging buffer may be rewritten only once the last copy out of it has run.  Every step ends
        with a synchronisation (the token read), which clears the mark; only a second upload without a
        step in between has to wait here."""
        if self._upload_pending:
            ops.stream_synchronize()
            self._upload_pending = False

    def _fill_tables(self) -> bool:
        """Write the requests' block tables into the staging buffer; True if they changed."""
        cache = self.engine.cache
        arr = self.host.numpy()
        changed = False
        for g, (a, b) in self._tables.items():
            state = [tuple(cache.requests[q].tables[g]) for q in self.requests]
            if self._table_state.get(g) == state:
                continue
            changed = True
            self._table_state[g] = state
            rows = cache.block_table(g, self.requests, self.widths[g])
            filler = [cache.pad_page[g]] + [RELEASED] * (self.widths[g] - 1)
            rows += [filler] * (self.batch - len(rows))
            arr[a:b] = np.asarray(rows, dtype=np.int32).reshape(-1)
        return changed

    def refresh_tables(self) -> None:
        """After the host reserved pages (or a window released some): bring the device tables up
        to date.  Only the table region travels."""
        cache = self.engine.cache
        if cache.tables_version == self._tables_version:
            return                                        # no table of the pool has changed since the last look
        self._tables_version = cache.tables_version
        if all(self._table_state.get(g) == [tuple(cache.requests[q].tables[g]) for q in self.requests]
               for g in self._tables):
            return
        self._wait_upload()
        if self._fill_tables():
            a = min(v[0] for v in self._tables.values())
            self.dev[a:self.total].copy_(self.host[a:self.total], non_blocking=True)
            self._mark_upload()

    def upload_tokens(self, tokens: Sequence[int]) -> None:
        """The host's copy of each request's next input token, pinned memory -> device.  A
        replay would find the same values where the sampler left them; sending them keeps the
        host the owner of what the model is fed."""
        self._wait_upload()
        if self._token_views is None:
            a, b = self._s["tokens"]
            if not self.host_io:
                ops.copy_async(self.dev[a:b], self.host[a:b])     # checked once; from now on by raw pointers
            self._token_views = (self.host.numpy()[a:b], self.host[a:b].data_ptr(), self.dev[a:b].data_ptr(), 4 * (b - a))
        array, pinned, device, nbytes = self._token_views
        array[:len(tokens)] = tokens
        if self.host_io:
            return                                        # the replay's first node copies them
        ops.copy_raw(device, pinned, nbytes, True)
        self._mark_upload()

    def stale(self, max_seq_len: int) -> bool:
        """The captured step was cut for another context length than the one it is about to serve."""
        return self.graph is not None and any(m.plan_stale(self.ctx, max_seq_len) for m in self._planners)

    def invalidate(self) -> None:
        """Forget the captured step and the launch plans frozen into it; the next capture plans anew."""
        self.graph = None
        for mixer in self._planners:
            mixer.forget_plans(self.ctx)

    def fits(self, requests: Sequence[Hashable]) -> bool:
        cache = self.engine.cache
        return all(len(cache.requests[q].tables[g]) <= w for g, w in self.widths.items() for q in requests)

    # ------------------------------------------------------------------ capture and replay
    def _body(self) -> None:
        if self.host_io:
            a, b = self._s["tokens"]
            ops.copy_raw(self.dev[a:b].data_ptr(), self.host[a:b].data_ptr(), 4 * (b - a), True)
        logits = self.engine.model.forward(self.ctx, self.views)
        ops.sample_rows(logits, self.temperature, self.top_k, self.seed, self.draw, self.ctx.token_ids)
        ops.decode_advance(self.ctx.positions, self.ctx.seq_pos0, self.ctx.seq_lens, self.draw, self.ctx.token_ids,
                           self.engine.error_flag, self.out_dev, self.grows)
        if self.host_io:
            ops.copy_raw(self.out_host.data_ptr(), self.out_dev.data_ptr(), 4 * (self.batch + 1), False)

    def capture(self) -> None:
        """Run the step once eagerly (plans launches, warms libraries), then record it.  The
        eager run really executes: callers `load()` the true state again afterwards."""
        side = torch.cuda.Stream(device=self.engine.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..kernels.build import LaunchCounter
        before = LaunchCounter.own
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._body()
        self.launches_per_replay = LaunchCounter.own - before      # kernels of this library in the graph

    def replay(self) -> None:
        self.graph.replay()
        self.replays += 1

    def read_tokens(self) -> List[int]:
        """The tokens the last replay selected (one device -> host copy, synchronising)."""
        A = self.batch
        if not self.host_io:
            ops.copy_raw(self.out_host.data_ptr(), self.out_dev.data_ptr(), 4 * (A + 1), False)
        ops.stream_synchronize()
        self._upload_pending = False                      # everything queued before has run
        host = self.out_host.tolist()
        if host[A]:
            self.engine.error_flag.zero_()
            raise StepError(device_error_text(host[A]))
        return host[:self.active]


# Batch sizes that steps are captured for.  A step of fewer requests runs in the next size up, the rows in
# between filled with sequences of one token that live in the cache's spare page: when requests end one by one
# (the tail of a burst), every few steps would otherwise want a capture of their own, which costs as much as
# several steps.  Beyond the list: multiples of 64.
BATCH_SIZES = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def captured_batch(requests: int, most: int) -> int:
    """The captured batch size that serves `requests` requests when the cache has `most` request slots."""
    size = next((b for b in BATCH_SIZES if b >= requests), -(-requests // 64) * 64)
    return max(requests, min(size, most))


class DecodeGraphPool:
    """Captured decode steps by batch size (one of BATCH_SIZES) and table width; built on first use.  At most
    `max_graphs` are kept (each owns its activations and a captured graph): the one used longest ago goes first."""

    def __init__(self, engine: Engine, max_graphs: int = 32, host_io: bool = False):
        self.engine, self.host_io = engine, bool(host_io)
        self.max_graphs = max(1, int(max_graphs))
        self.graphs: Dict[tuple, DecodeGraph] = {}          # insertion order = order of last use
        self.captures = 0

    def get(self, requests: Sequence[Hashable], headroom_tokens: int = 0) -> DecodeGraph:
        cache = self.engine.cache
        widths = {}
        for g in cache.groups:
            need = max(cache.blocks_for(cache.length(q) + 1 + headroom_tokens) for q in requests)
            need = max(need, max(len(cache.requests[q].tables[g]) for q in requests))
            widths[g] = max(8, _round_up_pow2(need))
        batch = captured_batch(len(requests), cache.max_requests)
        key = (batch, tuple(sorted(widths.items())))
        graph = self.graphs.pop(key, None)
        if graph is None:
            while len(self.graphs) >= self.max_graphs:
                del self.graphs[next(iter(self.graphs))]
            graph = DecodeGraph(self.engine, batch, widths, host_io=self.host_io)
        self.graphs[key] = graph                             # (re)inserted last: most recently used
        return graph

    def ensure_captured(self, graph: DecodeGraph) -> None:
        if graph.graph is None:
            graph.capture()
            self.captures += 1
