"""The Python entry point: a model folder in, tokens out.

`LLM.generate(prompts, config)` is the call a user makes; `submit` / `step` / `poll` /
`cancel` expose the scheduler for callers that feed requests over time.  Option names and
meanings are the reference's (`GenerationConfig`, include/microllm/inference/generator.h:11-23;
`submit`/`step`/`cancel` of its continuous scheduler, include/microllm/inference/scheduler.h:191-290).
Token ids travel host -> device once per step inside the step's metadata buffer; one small
device -> host copy per step brings the selected tokens (and the kernels' error flag) back.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..sampling.config import GenerationConfig
from ..sampling.sampler import Sampler
from .decode_graph import DecodeGraph, DecodeGraphPool, graph_capable
from .loading import DEFAULT_PAGE_SIZE, load_engine
from .scheduler import PENDING, Request, Scheduler, StepPlan
from .step import Engine, OutOfPages, StepEntry, StepError, device_error_text


class _Issued:
    """A step that was handed to the GPU and whose selected tokens have not been read yet: `packed` holds them on
    the device (and the error flag behind them), `host` is the pinned copy that `copied` says has arrived."""
    __slots__ = ("plan", "packed", "wanting", "host", "copied")

    def __init__(self, plan: StepPlan, packed: torch.Tensor, wanting: List[Request], host: torch.Tensor, copied):
        self.plan, self.packed, self.wanting, self.host, self.copied = plan, packed, wanting, host, copied


class LLM:
    def __init__(self, model: Union[str, Engine], dtype="bfloat16", page_size: int = DEFAULT_PAGE_SIZE,
                 num_pages: Optional[int] = None, max_tokens: Optional[int] = None, max_tokens_per_step: int = 2048,
                 max_seqs: int = 64, device: Optional[str] = None, cuda_graphs: bool = True):
        if isinstance(model, Engine):
            self.engine = model
        else:
            self.engine = load_engine(model, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                      max_tokens=max_tokens, max_requests=max_seqs, device=device,
                                      max_step_tokens=max_tokens_per_step)
        spec = self.engine.model.spec
        self.scheduler = Scheduler(self.engine.cache, spec.vocab_size, spec.max_position,
                                   max_tokens_per_step=max_tokens_per_step,
                                   max_seqs=min(max_seqs, self.engine.cache.max_requests))
        self.sampler = Sampler(self.engine.device)
        self.graphs = DecodeGraphPool(self.engine, host_io=True) if cuda_graphs and graph_capable(self.engine) else None
        self._graph: Optional[DecodeGraph] = None       # the captured step whose device state is current
        self.graph_steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.wait_s = 0.0            # host time spent blocked in the step's one device -> host read: the GPU was busy for all of it
        # Steady decoding: while the GPU runs a captured step the host already prepares the next one (pages, tables,
        # the check of the captured plan), so that between reading a step's tokens and launching the next step
        # only the scheduler's update and the token upload remain.  The prepared plan is used only if nothing
        # happened in between that the scheduler would have decided differently.
        self._prepared: Optional[StepPlan] = None
        self.prepared_steps = 0
        # ... and when the tokens just read change nothing about the batch (no stop token among them, nobody new waiting),
        # that step is launched before the scheduler's books are written: (plan, graph) of the replay on its way
        self._launched: Optional[tuple] = None
        self.launched_early = 0
        # Steps issued kernel by kernel: the one whose tokens are not read yet (see step())
        self._inflight: Optional[_Issued] = None
        self.lookahead = True
        self.lookahead_steps = 0
        # pinned landing places for the tokens of steps on their way (two are in use at most)
        self._results = [torch.empty(self.scheduler.max_seqs + 1, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._results_next = 0

    # ------------------------------------------------------------------ request interface
    def submit(self, prompt: Sequence[int], config: Optional[GenerationConfig] = None) -> int:
        return self.scheduler.submit(prompt, config)

    def cancel(self, request_id: int) -> bool:
        self._prepared = None
        return self.scheduler.cancel(request_id)

    def poll(self, request_id: int) -> Request:
        """The request's record: `state`, `reason`, `output` (the tokens generated so far), timings."""
        return self.scheduler.requests[request_id]

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None or self._launched is not None

    def step(self) -> List[Request]:
        """One scheduler decision, one model step, one token selection.  Returns the requests
        that finished in it.

        Steps that hold prompt portions are issued kernel by kernel, and the host has work to do around them
        (update, schedule, pack the metadata, issue the first layers).  So that the GPU does not idle meanwhile,
        the NEXT such step is planned and issued while this one runs, before this one's tokens are read: the
        requests that decode get a stand-in for their input token, and a small kernel behind this step's token
        selection puts the selected tokens in their places (Engine.step's `patch`).  What this call returns is
        still this step's outcome; a request that ends on a stop token has one void row in the step issued ahead.

        Captured decode steps: once a step's tokens are read and they change nothing about the batch, the next
        replay (prepared while this one ran) is launched with them before this call returns; the next call finds it
        on its way (`_launched`) and only has the bookkeeping and the read left."""
        if self._launched is not None:
            (plan, graph), self._launched = self._launched, None
            return self._graph_step(plan, launched=graph)
        if self._inflight is None:
            prepared, self._prepared = self._prepared, None
            if (prepared is not None and not self.scheduler.waiting and len(prepared.entries) == len(self.scheduler.running)
                    and all(e.request.computed == e.begin and not e.request.finished for e in prepared.entries)):
                return self._graph_step(prepared, prepared=True)
            plan = self.scheduler.schedule()
            if not plan.entries:
                if self.scheduler.has_work() and not plan.preempted:
                    raise StepError("the scheduler has work but could plan nothing: the page pool is too small")
                return []
            if self._captured(plan):
                return self._graph_step(plan)
            self._graph = None
            self._inflight = self._issue(plan, None)
        current, self._inflight = self._inflight, None
        ahead = self._issue_ahead(current)
        try:
            finished = self._collect(current)
        except Exception:
            self._abandon(current.plan, ahead.plan if ahead is not None else None)
            raise
        self._inflight = ahead
        return finished

    def _abandon(self, *plans: Optional[StepPlan]) -> None:
        """A step failed (a device error, logits that were not finite).  What it computed, and what a step issued on
        top of it computed, is not to be trusted, and their requests stand between two states (tokens counted as
        computed, a token still pending).  They end as cancelled and give their pages back, so that the books stay
        whole and the other requests, and new ones, go on."""
        self._inflight = self._graph = self._prepared = self._launched = None
        for plan in plans:
            for e in (plan.entries if plan is not None else ()):
                if not e.request.finished:
                    self.scheduler.cancel(e.request.id)

    def _captured(self, plan: StepPlan) -> bool:
        """Every request brings its one last-selected token and steps are captured: the plan is a replay."""
        return self.graphs is not None and not plan.preempted and all(
            e.count == 1 and e.wants_logits and e.begin >= len(e.request.prompt) for e in plan.entries)

    def _issue(self, plan: StepPlan, before) -> "_Issued":
        """Hand `plan` to the step function and select its tokens, all asynchronously.  `before`: the step issued
        just before it whose tokens are not read yet; input tokens that it selects are patched in on the device."""
        entries, pairs = [], []
        place = 0
        rows_before = {id(r): i for i, r in enumerate(before.wanting)} if before is not None else {}
        for e in plan.entries:
            tokens = e.request.tokens(e.begin, e.begin + e.count)
            for j, t in enumerate(tokens):
                if t == PENDING:
                    if id(e.request) not in rows_before:
                        raise StepError("a plan feeds a token that no step on its way selects")
                    tokens[j] = 0
                    pairs.append((place + j, rows_before[id(e.request)]))
            place += e.count
            entries.append(StepEntry(e.request.id, tokens, [e.count - 1] if e.wants_logits else []))
        logits = self.engine.step(entries, patch=(before.packed, pairs) if pairs else None)
        wanting = [e.request for e in plan.entries if e.wants_logits]
        R = len(wanting)
        packed = torch.empty(R + 1, dtype=torch.int32, device=self.engine.device)
        if R:
            # draws are counted without the tokens still on their way
            self.sampler.sample_into(logits, [r.config for r in wanting], [len(r.generated) for r in wanting], packed[:R])
        packed[R:].copy_(self.engine.error_flag)
        # the copy back is queued HERE, behind this step's selection: queued when the tokens are wanted it would
        # stand behind whatever was issued in between (the next step)
        host = self._results[self._results_next][:R + 1]
        self._results_next = (self._results_next + 1) % len(self._results)
        host.copy_(packed, non_blocking=True)
        copied = torch.cuda.Event()
        copied.record()
        self.scheduler.begin(plan)
        self.h2d_bytes += 4 * plan.num_tokens
        self.d2h_bytes += 4 * (R + 1)
        return _Issued(plan, packed, wanting, host, copied)

    def _issue_ahead(self, current: "_Issued") -> Optional["_Issued"]:
        """While `current` runs: plan and issue the step after it, if that is a step this path runs anyway (it holds
        a prompt portion, or steps are not captured) and nobody has to give up pages for it."""
        if not self.lookahead:
            return None
        sched = self.scheduler
        if self.graphs is not None and not sched.waiting and all(r.known - r.computed <= 1 for r in sched.running):
            return None                                   # what follows is steady decoding: captured steps take over
        if sched.would_preempt():
            return None
        plan = sched.schedule()
        if not plan.entries or plan.preempted or self._captured(plan):
            return None                                   # (reservations and admissions it made stand: the next schedule() finds them)
        try:
            issued = self._issue(plan, current)
        except OutOfPages:
            return None                                   # nothing was launched; the next schedule() decides who gives way
        self.lookahead_steps += 1
        return issued

    def _collect(self, issued: "_Issued") -> List[Request]:
        """Read the step's tokens (the one device -> host copy, blocking) and let the scheduler conclude it."""
        R = len(issued.wanting)
        t0 = time.perf_counter()
        issued.copied.synchronize()
        host = issued.host.tolist()
        self.wait_s += time.perf_counter() - t0
        if host[R]:
            self.engine.error_flag.zero_()
            raise StepError(device_error_text(host[R]))
        return self.scheduler.finish(issued.plan, host[:R])

    def _prepare_next(self, plan: StepPlan, graph: DecodeGraph) -> None:
        """While the GPU runs `plan` as a captured step: what the same requests' next step needs from the host.
        Leaves a plan in self._prepared only if that step can be this graph's next replay as it stands."""
        if self.scheduler.waiting or len(plan.entries) != len(self.scheduler.running) or len(plan.entries) > self.scheduler.max_seqs:
            return
        cache = self.engine.cache
        for e in plan.entries:
            if len(e.request.generated) + 2 > e.request.config.max_new_tokens:
                return                                   # ends by length with this step's token: the batch changes
            if not cache.reserve(e.request.id, e.begin + 2):
                return                                   # out of pages: the scheduler decides who gives way
        ids = graph.requests
        if graph.stale(max(e.begin for e in plan.entries) + 2) or not graph.fits(ids):
            return
        graph.refresh_tables()                           # queued behind the running step; the next replay finds them
        self._prepared = StepPlan([type(e)(e.request, e.begin + 1, 1, True) for e in plan.entries])

    def _graph_step(self, plan: StepPlan, prepared: bool = False, launched: Optional[DecodeGraph] = None) -> List[Request]:
        """A step in which every request brings its one last-selected token: replay the captured
        decode step instead of launching it kernel by kernel.  `launched`: the replay is on its way already (it was
        started at the end of the step before, see below); what remains is the bookkeeping and the read."""
        ids = [e.request.id for e in plan.entries]
        graph = self._graph
        longest = max(e.begin for e in plan.entries) + 1
        if launched is not None:
            graph = launched
        elif prepared and graph is not None and graph.requests == ids:
            # pages, tables and the captured plan were seen to while the last step ran
            graph.upload_tokens([e.request.token(e.begin) for e in plan.entries])
            self.h2d_bytes += 4 * graph.batch
            self.prepared_steps += 1
        else:
            if graph is not None and graph.stale(longest):
                graph = None                             # the context outgrew the way the captured step cuts the keys
            if graph is None or graph.requests != ids or not graph.fits(ids):
                remaining = max(e.request.config.max_new_tokens - len(e.request.generated) for e in plan.entries)
                graph = self.graphs.get(ids, headroom_tokens=remaining)
                if graph.stale(longest):
                    graph.invalidate()                   # captured for another context length: plan and capture anew
                state = ([e.request.token(e.begin) for e in plan.entries], [e.begin for e in plan.entries],
                         [e.request.config for e in plan.entries], [len(e.request.generated) for e in plan.entries])
                graph.load(ids, *state)
                if graph.graph is None:
                    self.graphs.ensure_captured(graph)
                    graph.load(ids, *state)              # the eager run before capture moved the state
                self._graph = graph
                self.h2d_bytes += 4 * graph.total
            else:
                graph.refresh_tables()
                graph.upload_tokens([e.request.token(e.begin) for e in plan.entries])
                self.h2d_bytes += 4 * graph.batch
        if launched is None:
            graph.replay()
        # what does not need the step's tokens happens while the GPU runs
        for e in plan.entries:
            if not e.request.finished:                   # (cancelled since a replay launched early took it along)
                self.engine.cache.commit(e.request.id, e.begin + 1)
        self._prepare_next(plan, graph)
        self.d2h_bytes += 4 * (graph.batch + 1)
        self.graph_steps += 1
        self.engine.steps_run += 1
        self.engine.tokens_run += len(ids)
        t0 = time.perf_counter()
        try:
            tokens = graph.read_tokens()
        except StepError:
            self._abandon(plan)
            raise
        self.wait_s += time.perf_counter() - t0
        # The next replay is prepared and these tokens change nothing about the batch (no stop token, nobody ended by
        # length or it would not be prepared, nobody new waiting): it starts NOW, fed with the tokens just read, and
        # the scheduler's books are written while it runs.  The next step() finds it on its way.
        ahead = self._prepared
        if (ahead is not None and self.lookahead and not self.scheduler.waiting and self._graph is graph and
                all(t >= 0 and t not in e.request.config.stop_tokens for e, t in zip(plan.entries, tokens))):
            graph.upload_tokens(tokens)
            graph.replay()
            self.h2d_bytes += 4 * graph.batch
            self.prepared_steps += 1
            self.launched_early += 1
            self._prepared, self._launched = None, (ahead, graph)
        try:
            finished = self.scheduler.update(plan, tokens)
        except Exception:
            self._abandon(plan)
            raise
        if finished:
            self._graph = None
            self._prepared = None
        return finished

    # ------------------------------------------------------------------ whole generations
    def generate(self, prompts: Sequence[Sequence[int]],
                 config: Union[GenerationConfig, Sequence[GenerationConfig], None] = None) -> List[List[int]]:
        """Generate for every prompt (token ids); returns the new tokens of each, in order."""
        if prompts and isinstance(prompts[0], int):
            raise TypeError("generate takes a list of prompts, each a list of token ids")
        configs = list(config) if isinstance(config, (list, tuple)) else [config or GenerationConfig()] * len(prompts)
        if len(configs) != len(prompts):
            raise ValueError("one GenerationConfig per prompt, or one for all")
        ids = [self.submit(p, c) for p, c in zip(prompts, configs)]
        while self.has_work():
            self.step()
        out = [list(self.scheduler.requests[i].generated) for i in ids]
        for i in ids:
            del self.scheduler.requests[i]
        return out

    generate_batch = generate

    def metrics(self) -> Dict[str, object]:
        m = dict(vars(self.scheduler.metrics))
        m["cache"] = self.engine.cache.stats()
        return m
