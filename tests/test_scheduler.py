"""The scheduler's decisions, driven by a fake step on the host: admission order, portions
under the token budget, decode beside prompts, finishing, cancelling, and what happens when
pages run out."""
import pytest

from microllm_rocm_b200.cache import CacheManager
from microllm_rocm_b200.engine.scheduler import PENDING, FinishReason, RequestState, Scheduler
from microllm_rocm_b200.parts.base import PagedKVNeed
from microllm_rocm_b200.sampling import GenerationConfig

VOCAB = 50


def next_token(prefix):
    """The fake model: the token after `prefix` is a pure function of the prefix."""
    h = 7
    for t in prefix:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


def oracle(prompt, cfg):
    seq, out = list(prompt), []
    for _ in range(cfg.max_new_tokens):
        t = next_token(seq)
        out.append(t); seq.append(t)
        if t in cfg.stop_tokens:
            break
    return out


class Harness:
    def __init__(self, num_pages=64, page_size=4, max_requests=8, budget=16, max_seqs=8, window=None):
        entries = {"l0": PagedKVNeed(1, 8, None)}
        if window:
            entries["l1"] = PagedKVNeed(1, 8, window)
        self.cache = CacheManager(entries, page_size, num_pages, max_requests)
        self.s = Scheduler(self.cache, VOCAB, 4096, max_tokens_per_step=budget, max_seqs=max_seqs)
        self.fed = {}                      # request id -> tokens the "cache" holds
        self.plans = []

    def step(self):
        plan = self.s.schedule()
        for rid in plan.preempted:
            self.fed.pop(rid, None)
        drawn = []
        for e in plan.entries:
            r = e.request
            held = self.fed.setdefault(r.id, [])
            assert len(held) == e.begin == self.cache.length(r.id), "a portion must continue where the cache ends"
            held.extend(r.tokens(e.begin, e.begin + e.count))
            self.cache.commit(r.id, e.begin + e.count)
            if e.wants_logits:
                assert len(held) == r.known
                drawn.append(next_token(held))
        self.cache.check()
        self.plans.append(plan)
        done = self.s.update(plan, drawn)
        for r in done:
            self.fed.pop(r.id, None)
        return plan, done

    def run(self, limit=10000):
        n = 0
        while self.s.has_work():
            self.step()
            n += 1
            assert n < limit, "the scheduler makes no progress"
        return n


def test_tokens_equal_the_serial_oracle_for_any_mix():
    h = Harness(budget=16)
    prompts = [[1, 2, 3], list(range(40)), [9] * 17, [4, 4], list(range(30, 45))]
    cfgs = [GenerationConfig(max_new_tokens=n, temperature=0.0) for n in (5, 9, 1, 12, 7)]
    ids = [h.s.submit(p, c) for p, c in zip(prompts, cfgs)]
    h.run()
    for i, p, c in zip(ids, prompts, cfgs):
        r = h.s.requests[i]
        assert r.generated == oracle(p, c) and r.state == RequestState.COMPLETED and r.reason == FinishReason.LENGTH
    assert h.cache.stats()["full"]["used"] == 0 and not h.cache.requests
    m = h.s.metrics
    assert m.admissions == 5 and m.completions == 5 and m.preemptions == 0
    assert m.tokens_generated == sum(c.max_new_tokens for c in cfgs)
    assert m.max_tokens_in_step <= 16


def test_budget_cuts_prompts_into_portions_and_decodes_beside_them():
    h = Harness(budget=8)
    a = h.s.submit([1, 2, 3], GenerationConfig(max_new_tokens=6, temperature=0.0))
    plan, _ = h.step()
    assert [(e.request.id, e.begin, e.count, e.wants_logits) for e in plan.entries] == [(a, 0, 3, True)]
    b = h.s.submit(list(range(20)), GenerationConfig(max_new_tokens=2, temperature=0.0))
    plan, _ = h.step()        # a decodes one token, b gets the remaining 7 of the budget
    assert [(e.request.id, e.begin, e.count, e.wants_logits) for e in plan.entries] == [(a, 3, 1, True), (b, 0, 7, False)]
    plan, _ = h.step()
    assert [(e.request.id, e.begin, e.count, e.wants_logits) for e in plan.entries] == [(a, 4, 1, True), (b, 7, 7, False)]
    plan, _ = h.step()
    assert [(e.request.id, e.begin, e.count, e.wants_logits) for e in plan.entries] == [(a, 5, 1, True), (b, 14, 6, True)]
    assert h.s.requests[b].first_token_step == 3
    h.run()
    assert h.s.requests[b].generated == oracle(list(range(20)), GenerationConfig(max_new_tokens=2, temperature=0.0))


def test_admission_is_fifo_and_waits_for_slots_and_pages_without_preempting():
    h = Harness(num_pages=6, page_size=4, max_requests=2, budget=64)
    ids = [h.s.submit([i] * 8, GenerationConfig(max_new_tokens=4, temperature=0.0)) for i in range(4)]
    plan, _ = h.step()
    assert [e.request.id for e in plan.entries] == ids[:2], "two slots: two admitted, in order"
    assert h.s.metrics.preemptions == 0
    h.run()
    order = [i for p in h.plans for i in [e.request.id for e in p.entries if e.begin == 0]]
    assert order == ids
    assert all(h.s.requests[i].generated == oracle([k] * 8, GenerationConfig(max_new_tokens=4, temperature=0.0))
               for k, i in enumerate(ids))


def test_running_out_of_pages_preempts_the_youngest_and_recomputes():
    # 5 pages of 4 tokens; two requests of 8 tokens fit (4 pages) but cannot both grow to 13
    h = Harness(num_pages=5, page_size=4, max_requests=4, budget=64)
    cfg = GenerationConfig(max_new_tokens=6, temperature=0.0)
    a = h.s.submit([1] * 8, cfg)
    b = h.s.submit([2] * 8, cfg)
    h.step()                                   # both prefilled: 4 pages held
    plan, _ = h.step()                         # each needs a 3rd page; only one is free
    assert plan.preempted == [b] and [e.request.id for e in plan.entries] == [a]
    assert h.s.requests[b].state == RequestState.WAITING and h.s.requests[b].computed == 0
    assert h.s.waiting[0].id == b and len(h.s.requests[b].generated) == 1, "what it generated stays known"
    h.run()
    assert h.s.requests[a].generated == oracle([1] * 8, cfg)
    assert h.s.requests[b].generated == oracle([2] * 8, cfg), "recomputation continues the same sequence"
    assert h.s.metrics.preemptions >= 1 and h.s.requests[b].preemptions >= 1
    # b came back as an ordinary prompt of prompt + generated tokens
    back = [e for p in h.plans[2:] for e in p.entries if e.request.id == b and e.begin == 0][0]
    assert back.count > 8
    assert h.cache.stats()["full"]["used"] == 0


def test_a_request_that_can_never_fit_is_refused_at_submit():
    h = Harness(num_pages=4, page_size=4)
    with pytest.raises(ValueError, match="could never run"):
        h.s.submit([1] * 10, GenerationConfig(max_new_tokens=8))
    h.s.submit([1] * 10, GenerationConfig(max_new_tokens=7, temperature=0.0))      # 16 cached tokens: fits exactly
    h.run()
    s2 = Scheduler(h.cache, VOCAB, 12)
    with pytest.raises(ValueError, match="exceeds model context"):
        s2.submit([1] * 10, GenerationConfig(max_new_tokens=3))


def test_submit_validation_follows_the_reference():
    h = Harness()
    for prompt, cfg, word in [([], GenerationConfig(), "empty"), ([VOCAB], GenerationConfig(), "vocabulary"),
                              ([1], GenerationConfig(max_new_tokens=-1), "non-negative"),
                              ([1], GenerationConfig(temperature=-0.5), "temperature"),
                              ([1], GenerationConfig(temperature=float("nan")), "temperature"),
                              ([1], GenerationConfig(top_k=VOCAB + 1), "top_k"),
                              ([1], GenerationConfig(stop_tokens=(3, 3)), "unique"),
                              ([1], GenerationConfig(stop_tokens=(VOCAB,)), "stop token")]:
        with pytest.raises(ValueError, match=word):
            h.s.submit(prompt, cfg)
    rid = h.s.submit([1, 2], GenerationConfig(max_new_tokens=0))
    assert h.s.requests[rid].state == RequestState.COMPLETED and not h.s.has_work()


def test_stop_token_is_appended_then_ends_and_frees():
    prompt = [3, 1, 4]
    full = oracle(prompt, GenerationConfig(max_new_tokens=10, temperature=0.0))
    stop = full[3]
    cfg = GenerationConfig(max_new_tokens=10, temperature=0.0, stop_tokens=(stop,))
    h = Harness()
    rid = h.s.submit(prompt, cfg)
    h.run()
    r = h.s.requests[rid]
    want = full[:full.index(stop) + 1]
    assert r.generated == want and r.reason == FinishReason.STOP_TOKEN
    assert not h.cache.requests


def test_cancel_frees_at_once_whether_waiting_or_running():
    h = Harness(max_requests=1)
    a = h.s.submit([1] * 6, GenerationConfig(max_new_tokens=20, temperature=0.0))
    b = h.s.submit([2] * 6, GenerationConfig(max_new_tokens=20, temperature=0.0))
    h.step()
    assert h.s.cancel(b) and h.s.requests[b].reason == FinishReason.CANCELLED
    assert h.s.cancel(a) and not h.cache.requests and not h.s.has_work()
    assert not h.s.cancel(a)
    assert h.s.metrics.cancellations == 2


def test_window_group_lets_a_long_request_run_in_a_small_pool():
    # full group needs all pages; this only checks that planning works with two groups
    h = Harness(num_pages=16, page_size=4, window=8, budget=12)
    cfg = GenerationConfig(max_new_tokens=20, temperature=0.0)
    rid = h.s.submit(list(range(30)), cfg)
    h.run()
    assert h.s.requests[rid].generated == oracle(list(range(30)), cfg)
    assert h.cache.pages_released_by_window > 0


@pytest.mark.parametrize("seed", range(12))
def test_random_arrivals_cancellations_and_tight_pools_keep_the_books_and_the_tokens(seed):
    """Random prompts, lengths, stop tokens, arrival times and cancellations against pools of random
    tightness (some with a window group): after every step the cache's books are consistent; every request
    that was not cancelled ends with exactly the oracle's tokens, whatever was preempted and recomputed on
    the way; in the end nothing is held."""
    import random
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    longest = 60
    window = rng.choice([None, None, 8, 16])
    pages = rng.randint(-(-(longest + 24) // page) + 1, 3 * (longest + 24) // page)
    h = Harness(num_pages=pages, page_size=page, max_requests=rng.randint(2, 6), budget=rng.choice([3, 8, 16, 64]),
                max_seqs=rng.randint(2, 6), window=window)
    todo = []
    for _ in range(25):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.randint(1, longest))]
        stops = tuple(rng.sample(range(VOCAB), rng.choice([0, 0, 3])))
        todo.append((prompt, GenerationConfig(max_new_tokens=rng.randint(0, 24), temperature=0.0, stop_tokens=stops)))
    submitted, cancelled = [], set()
    steps = 0
    while todo or h.s.has_work():
        for _ in range(rng.randrange(0, 3)):
            if todo:
                prompt, cfg = todo.pop()
                submitted.append((h.s.submit(prompt, cfg), prompt, cfg))
        if submitted and rng.random() < 0.08:
            rid = rng.choice(submitted)[0]
            if h.s.requests[rid].state in (RequestState.WAITING, RequestState.RUNNING) and h.s.cancel(rid):
                cancelled.add(rid)
                h.fed.pop(rid, None)
        if h.s.has_work():
            h.step()
        steps += 1
        assert steps < 20000, "the scheduler makes no progress"
    for rid, prompt, cfg in submitted:
        r = h.s.requests[rid]
        if rid in cancelled:
            assert r.state == RequestState.CANCELLED and r.generated == oracle(prompt, cfg)[:len(r.generated)]
        else:
            assert r.state == RequestState.COMPLETED and r.generated == oracle(prompt, cfg), (rid, r.preemptions)
    h.cache.check()
    stats = h.cache.stats()
    assert not h.cache.requests and all(stats[g]["used"] == 0 for g in h.cache.groups)


class PipelinedHarness(Harness):
    """The same fake step, but driven the way LLM.step drives it: a plan is begun when it is issued, the NEXT plan
    is made and issued before the first one's tokens are read (unless pages would have to be taken from somebody),
    and only then the first is finished.  A fed token that is still PENDING is looked up in the results of the
    plan before, as the device-side patch does."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.inflight = None
        self.issued_ahead = 0
        self.void_rows = 0

    def issue(self, plan, before):
        from microllm_rocm_b200.engine.scheduler import PENDING
        for rid in plan.preempted:
            self.fed.pop(rid, None)
        drawn = []
        for e in plan.entries:
            r = e.request
            held = self.fed.setdefault(r.id, [])
            assert len(held) == e.begin == self.cache.length(r.id), "a portion must continue where the cache ends"
            tokens = r.tokens(e.begin, e.begin + e.count)
            for j, t in enumerate(tokens):
                if t == PENDING:
                    assert before is not None and r.id in before[2], "a pending token must come from the plan on its way"
                    tokens[j] = before[2][r.id]
            held.extend(tokens)
            self.cache.commit(r.id, e.begin + e.count)
            if e.wants_logits:
                drawn.append(next_token(held))
        self.cache.check()
        self.plans.append(plan)
        by_request = {e.request.id: t for e, t in zip([e for e in plan.entries if e.wants_logits], drawn)}
        self.s.begin(plan)
        return plan, drawn, by_request

    def step(self):
        if self.inflight is None:
            plan = self.s.schedule()
            if not plan.entries:
                return plan, []
            self.inflight = self.issue(plan, None)
        current, self.inflight = self.inflight, None
        ahead = None
        if not self.s.would_preempt():
            plan2 = self.s.schedule()
            if plan2.entries and not plan2.preempted:
                ahead = self.issue(plan2, current)
                self.issued_ahead += 1
        live_before = {e.request.id for e in current[0].entries if not e.request.finished}
        done = self.s.finish(current[0], current[1])
        self.void_rows += sum(1 for e in current[0].entries if e.request.id not in live_before)
        for r in done:
            self.fed.pop(r.id, None)
        self.inflight = ahead
        return current[0], done

    def run(self, limit=10000):
        n = 0
        while self.s.has_work() or self.inflight is not None:
            self.step()
            n += 1
            assert n < limit, "the scheduler makes no progress"
        return n


@pytest.mark.parametrize("pages,budget", [(64, 16), (64, 5), (9, 16), (8, 7)])
def test_plans_made_ahead_of_their_predecessors_results_give_the_same_tokens(pages, budget):
    """With every plan issued before the plan before it is finished: the tokens of every request are still the
    serial oracle's, also when requests end on stop tokens (their row in the plan issued ahead is void), when the
    pool is so tight that running requests are preempted (no plan is made ahead then), and with cancels and
    arrivals in between; nothing is left in the cache."""
    import random
    from microllm_rocm_b200.engine.scheduler import PENDING
    rng = random.Random(pages * 100 + budget)
    h = PipelinedHarness(num_pages=pages, page_size=4, max_requests=4, budget=budget, max_seqs=4)
    specs = []
    for i in range(14):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.choice([1, 2, 5, 9, 17]))]
        cfg = GenerationConfig(max_new_tokens=rng.choice([1, 2, 6, 11]), temperature=0.0,
                               stop_tokens=tuple(rng.sample(range(VOCAB), 6)) if i % 2 else ())
        specs.append((prompt, cfg))
    todo, ids, cancelled = list(specs), [], set()
    n = 0
    while todo or h.s.has_work() or h.inflight is not None:
        for _ in range(rng.randrange(0, 3) if pages > 9 else len(todo)):      # a tight pool gets the whole burst at once
            if todo:
                ids.append(h.s.submit(*todo.pop(0)))
        if ids and rng.random() < 0.08:
            victim = rng.choice(ids)
            if h.s.cancel(victim):
                cancelled.add(victim)
                h.fed.pop(victim, None)
        h.step()
        n += 1
        assert n < 5000
    for rid, (prompt, cfg) in zip(ids, specs):
        r = h.s.requests[rid]
        assert PENDING not in r.generated
        want = oracle(prompt, cfg)
        if rid in cancelled:
            assert r.generated == want[:len(r.generated)] and r.state == RequestState.CANCELLED
        else:
            assert r.generated == want, rid
            assert r.reason == (FinishReason.STOP_TOKEN if r.generated[-1] in cfg.stop_tokens else FinishReason.LENGTH)
    assert not h.cache.requests and h.cache.stats()["full"]["used"] == 0
    assert h.issued_ahead > 5
    if pages <= 9:
        assert h.s.metrics.preemptions > 0


def test_a_request_that_ends_on_a_stop_token_leaves_a_void_row_in_the_plan_issued_ahead():
    h = PipelinedHarness(budget=16)
    prompt = [3, 1, 4]
    full = oracle(prompt, GenerationConfig(max_new_tokens=8, temperature=0.0))
    stop = full[2]
    a = h.s.submit(prompt, GenerationConfig(max_new_tokens=8, temperature=0.0, stop_tokens=(stop,)))
    b = h.s.submit([7] * 5, GenerationConfig(max_new_tokens=8, temperature=0.0))
    h.run()
    assert h.s.requests[a].generated == full[:full.index(stop) + 1] and h.s.requests[a].reason == FinishReason.STOP_TOKEN
    assert h.s.requests[b].generated == oracle([7] * 5, GenerationConfig(max_new_tokens=8, temperature=0.0))
    assert h.void_rows == 1 and h.s.metrics.tokens_generated == len(h.s.requests[a].generated) + 8


def test_a_plan_whose_request_was_cancelled_before_it_began_leaves_that_request_alone():
    """A captured step may be launched for a plan before the books know of it; a request cancelled in between has a
    void row: beginning and finishing the plan must not count tokens for it nor leave a pending token behind."""
    h = Harness(budget=16)
    a = h.s.submit([3, 1, 4], GenerationConfig(max_new_tokens=8, temperature=0.0))
    b = h.s.submit([7] * 5, GenerationConfig(max_new_tokens=8, temperature=0.0))
    h.step()                                   # both prompts, first tokens
    plan = h.s.schedule()                      # both decode
    assert [e.request.id for e in plan.entries] == [a, b] and all(e.count == 1 for e in plan.entries)
    before = list(h.s.requests[a].generated)
    assert h.s.cancel(a)
    h.s.begin(plan)
    assert h.s.requests[a].generated == before and PENDING not in h.s.requests[a].generated
    held = h.fed[b] + h.s.requests[b].tokens(plan.entries[1].begin, plan.entries[1].begin + 1)
    h.cache.commit(b, plan.entries[1].begin + 1)
    done = h.s.finish(plan, [0, next_token(held)])           # row 0 is void: whatever it selected is dropped
    assert done == [] and h.s.requests[a].generated == before
    assert h.s.requests[b].generated[-1] == next_token(held) and PENDING not in h.s.requests[b].generated
    h.fed[b] = held
    h.fed.pop(a)
    h.run()
    assert h.s.requests[b].generated == oracle([7] * 5, GenerationConfig(max_new_tokens=8, temperature=0.0))
    h.cache.check()
