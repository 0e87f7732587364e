"""The scheduler: admits requests, cuts prompts into portions under a token budget, puts
them beside the decode tokens of running requests, finishes and frees.  It decides, the
step function runs; it touches no device memory and can be driven by a fake step.

Every request is a list of known tokens (prompt + what was generated) and a count of how
many of them are in the cache.  A step feeds the next `n` known tokens of some requests;
logits are wanted exactly where a portion reaches the end of the known tokens, and the
token drawn there becomes known.  A decode step is the case n == 1; recomputation after a
preemption is an ordinary prompt.

Decisions:
  * order: running requests first, in admission order, then waiting ones in submission
    order; decode tokens cost 1 of the budget each, prompts take what is left.
  * admission needs a state slot and pages for the portion; if either is missing the request
    waits (nobody is preempted to admit).
  * when a RUNNING request cannot get the page for its next token, the most recently
    admitted running request is preempted: everything it holds is given back and it returns
    to the FRONT of the waiting queue, to be recomputed from its known tokens.  A request
    whose prompt + max_new_tokens can never fit the pool alone is refused at submit, so one
    request always makes progress.
  * a request finishes on a stop token (appended first) or at max_new_tokens, and gives
    back its pages and slot in the same step.
  * a plan may be made before the results of the plan before it are read: begin(plan) records what a plan that
    was handed to the step function WILL have done (its tokens are in the cache; where logits are wanted one
    more token is known, its value still PENDING), schedule() plans on from there, finish(plan, tokens) names
    the pending tokens and ends requests.  A request that ends on a stop token may then already sit in the next
    plan; that entry is void and finish() skips it.  update() is begin() and finish() in one.

The reference's continuous scheduler (src/inference/scheduler.cpp:464-1069) has fixed slots
with capacity reserved up front, admits only prompts of equal length together and prefills
them whole (:710-788), and therefore never runs out of memory mid-flight; request states,
validation at submit (:32-63, 853-883), finish reasons and metrics (scheduler.h:15-57,
161-189) are kept.
"""
from __future__ import annotations

import enum
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from ..sampling.config import GenerationConfig


PENDING = -1        # stands in `generated` for a token that a step on its way will select


class RequestState(enum.Enum):
    WAITING = "waiting"            # no tokens in the cache (new, or preempted)
    RUNNING = "running"            # holds cache; prefilling or decoding
    COMPLETED = "completed"
    CANCELLED = "cancelled"


class FinishReason(enum.Enum):
    NONE = "none"
    LENGTH = "length"
    STOP_TOKEN = "stop_token"
    CANCELLED = "cancelled"


@dataclass
class Request:
    id: int
    prompt: List[int]
    config: GenerationConfig
    state: RequestState = RequestState.WAITING
    reason: FinishReason = FinishReason.NONE
    generated: List[int] = field(default_factory=list)
    computed: int = 0                   # known tokens already in the cache
    arrival_step: int = 0
    first_token_step: Optional[int] = None
    completion_step: Optional[int] = None
    submitted_at: float = 0.0
    first_token_at: Optional[float] = None
    completed_at: Optional[float] = None
    preemptions: int = 0

    @property
    def known(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def output(self) -> List[int]:
        """The tokens generated so far.  (`generated` may end in PENDING entries while a step that will name them
        is on its way; a reader between steps wants this list.)"""
        return [t for t in self.generated if t != PENDING]

    def token(self, i: int) -> int:
        return self.prompt[i] if i < len(self.prompt) else self.generated[i - len(self.prompt)]

    def tokens(self, begin: int, end: int) -> List[int]:
        return [self.token(i) for i in range(begin, end)]

    @property
    def finished(self) -> bool:
        return self.state in (RequestState.COMPLETED, RequestState.CANCELLED)


@dataclass
class PlannedEntry:
    request: Request
    begin: int                      # first known token fed
    count: int
    wants_logits: bool              # the portion reaches the end of the known tokens


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[int] = field(default_factory=list)
    begun: bool = False             # begin() has recorded it as on its way

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


@dataclass
class SchedulerMetrics:
    steps: int = 0
    admissions: int = 0
    preemptions: int = 0
    completions: int = 0
    cancellations: int = 0
    prompt_tokens: int = 0          # tokens fed in portions longer than one, or without a draw
    decode_tokens: int = 0
    tokens_generated: int = 0
    max_tokens_in_step: int = 0
    max_seqs_in_step: int = 0


class Scheduler:
    def __init__(self, cache, vocab_size: int, max_position: int, max_tokens_per_step: int = 2048,
                 max_seqs: int = 64):
        if max_tokens_per_step <= 0 or max_seqs <= 0:
            raise ValueError("max_tokens_per_step and max_seqs must be positive")
        self.cache = cache
        self.vocab_size, self.max_position = int(vocab_size), int(max_position)
        self.max_tokens_per_step, self.max_seqs = int(max_tokens_per_step), int(max_seqs)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []            # in admission order
        self.requests: Dict[int, Request] = {}
        self.metrics = SchedulerMetrics()
        self._next_id = 0
        self.step_index = 0

    # ------------------------------------------------------------------ submit / cancel
    def capacity_tokens(self) -> int:
        return self.cache.num_pages * self.cache.page_size

    def submit(self, prompt: Sequence[int], config: Optional[GenerationConfig] = None) -> int:
        config = config or GenerationConfig()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("generation prompt cannot be empty")
        config.validate(self.vocab_size)
        for t in prompt:
            if not 0 <= t < self.vocab_size:
                raise ValueError("prompt token is outside the vocabulary")
        total = len(prompt) + config.max_new_tokens
        if total > self.max_position:
            raise ValueError("prompt plus generated tokens exceeds model context")
        # the last generated token is never fed back, so it needs no page
        if max(len(prompt), total - 1) > self.capacity_tokens():
            raise ValueError(f"request needs {total - 1} cached tokens but the page pool holds "
                             f"{self.capacity_tokens()}: it could never run")
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, prompt, config, arrival_step=self.step_index, submitted_at=time.perf_counter())
        self.requests[rid] = req
        if config.max_new_tokens == 0:                   # completes at once (scheduler.cpp:873-880)
            self._finish(req, FinishReason.LENGTH)
        else:
            self.waiting.append(req)
        return rid

    def cancel(self, rid: int) -> bool:
        req = self.requests.get(rid)
        if req is None or req.finished:
            return False
        if req in self.running:
            self.running.remove(req)
            self.cache.release(req.id)
        else:
            self.waiting.remove(req)
        req.state, req.reason = RequestState.CANCELLED, FinishReason.CANCELLED
        req.completion_step, req.completed_at = self.step_index, time.perf_counter()
        req.generated = [t for t in req.generated if t != PENDING]
        self.metrics.cancellations += 1
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning a step
    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.running.remove(req)
        self.cache.release(req.id)
        req.state, req.computed = RequestState.WAITING, 0
        req.preemptions += 1
        self.waiting.appendleft(req)
        self.metrics.preemptions += 1
        plan.preempted.append(req.id)
        plan.entries = [e for e in plan.entries if e.request is not req]

    def schedule(self) -> StepPlan:
        """Decide what the next step runs.  Reserves the pages it needs."""
        plan = StepPlan([])
        budget = self.max_tokens_per_step
        # 1. running requests, oldest first; the youngest is preempted when pages run out
        i = 0
        while i < len(self.running):
            req = self.running[i]
            if len(plan.entries) >= self.max_seqs or budget <= 0:
                break
            if req.computed >= req.known or self._ends_with_pending(req):
                i += 1                                    # nothing to feed: its last token is on its way
                continue
            count = min(req.known - req.computed, budget)
            while not self.cache.reserve(req.id, req.computed + count):
                victim = self.running[-1]
                self._preempt(victim, plan)
                if victim is req:
                    break
            else:
                plan.entries.append(PlannedEntry(req, req.computed, count, req.computed + count == req.known))
                budget -= count
                i += 1
                continue
            # req itself was preempted: the list shrank, the same index is the next request
            budget = self.max_tokens_per_step - plan.num_tokens
        # 2. waiting requests in order, while slots, pages and budget last
        while self.waiting and budget > 0 and len(plan.entries) < self.max_seqs and not plan.preempted:
            req = self.waiting[0]
            count = min(req.known - req.computed, budget)
            if not self.cache.add(req.id):
                break                                     # no state slot: wait
            if not self.cache.reserve(req.id, count):
                self.cache.release(req.id)
                break                                     # no pages: wait, preempt nobody
            self.waiting.popleft()
            req.state = RequestState.RUNNING
            self.running.append(req)
            self.metrics.admissions += 1
            plan.entries.append(PlannedEntry(req, 0, count, count == req.known))
            budget -= count
        return plan

    # ------------------------------------------------------------------ around the step
    @staticmethod
    def _ends_with_pending(req: Request) -> bool:
        """The request's last allowed token is being computed: nothing more may be planned for it."""
        return bool(req.generated) and req.generated[-1] == PENDING and len(req.generated) >= req.config.max_new_tokens

    def would_preempt(self) -> bool:
        """Whether the next schedule() might have to take pages from a running request: the pools cannot give every
        running request the pages of its next portion.  (A plan made ahead of its predecessor's results must not
        preempt: the victim's latest token is not known yet.)"""
        budget = self.max_tokens_per_step
        need: Dict[str, int] = {}
        seqs = 0
        for req in self.running:
            if seqs >= self.max_seqs or budget <= 0:
                break
            if req.computed >= req.known or self._ends_with_pending(req):
                continue
            count = min(req.known - req.computed, budget)
            for group, pages in self.cache.pages_needed(req.id, req.computed + count).items():
                need[group] = need.get(group, 0) + pages
            budget -= count
            seqs += 1
        return any(pages > self.cache.groups[group].pool.free_count for group, pages in need.items())

    def begin(self, plan: StepPlan) -> None:
        """`plan` has been handed to the step function: record what it will have done, so that the next plan can be
        made before its results are read."""
        if plan.begun:
            return
        for e in plan.entries:
            if e.request.finished:
                continue                  # cancelled after the plan was made: its row runs for nothing
            e.request.computed = e.begin + e.count
            if e.wants_logits:
                e.request.generated.append(PENDING)
        plan.begun = True

    def finish(self, plan: StepPlan, drawn: Sequence[int]) -> List[Request]:
        """`drawn` are the tokens selected at the plan's wanted rows (in plan order): name the pending tokens, end
        requests.  Returns the requests that finished."""
        if not plan.begun:
            self.begin(plan)
        finished: List[Request] = []
        now = time.perf_counter()
        it = iter(drawn)
        m = self.metrics
        m.steps += 1
        m.max_tokens_in_step = max(m.max_tokens_in_step, plan.num_tokens)
        m.max_seqs_in_step = max(m.max_seqs_in_step, len(plan.entries))
        for e in plan.entries:
            req = e.request
            token = int(next(it)) if e.wants_logits else None
            if req.finished:
                continue                  # ended (a stop token of the plan before, a cancel) while this plan was on its way
            if e.count == 1 and e.wants_logits and e.begin >= len(req.prompt):
                m.decode_tokens += 1
            else:
                m.prompt_tokens += e.count
            if token is None:
                continue
            if token < 0:
                raise RuntimeError(f"request {req.id}: logits were not finite, no token could be selected")
            req.generated[req.generated.index(PENDING)] = token
            m.tokens_generated += 1
            if req.first_token_step is None:
                req.first_token_step, req.first_token_at = self.step_index, now
            made = len(req.generated) - req.generated.count(PENDING)
            if token in req.config.stop_tokens:
                self._finish(req, FinishReason.STOP_TOKEN)
            elif made >= req.config.max_new_tokens:
                self._finish(req, FinishReason.LENGTH)
            if req.finished:
                finished.append(req)
        self.step_index += 1
        return finished

    def update(self, plan: StepPlan, drawn: Sequence[int]) -> List[Request]:
        """Record that `plan` ran and that `drawn` are the tokens selected at its wanted rows
        (in plan order).  Returns the requests that finished."""
        self.begin(plan)
        return self.finish(plan, drawn)

    def _finish(self, req: Request, reason: FinishReason) -> None:
        if req in self.running:
            self.running.remove(req)
            self.cache.release(req.id)
        req.state, req.reason = RequestState.COMPLETED, reason
        req.completion_step, req.completed_at = self.step_index, time.perf_counter()
        req.generated = [t for t in req.generated if t != PENDING]       # what a plan on its way would have added
        self.metrics.completions += 1
