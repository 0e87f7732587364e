"""A fixed batch of requests in steady decode, for measurement: prompts are prefilled in
portions, then every `step()` feeds each request the token it was given last and selects
the next one greedily.  Counted tokens equal forward passes, as in the reference's steady
decode accounting (apps/hf_infer.cpp:1464-1468)."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from ..kernels.build import LaunchCounter
from ..sampling.config import GenerationConfig
from .decode_graph import DecodeGraphPool, graph_capable
from .step import Engine, StepEntry


class DecodeSession:
    def __init__(self, engine: Engine, prompts: Sequence[Sequence[int]], max_steps: int, prefill_budget: int = 2048,
                 use_graph: bool = True):
        self.engine = engine
        self.ids = [f"bench{i}" for i in range(len(prompts))]
        cache = engine.cache
        for rid in self.ids:
            if not cache.add(rid):
                raise RuntimeError("not enough request slots for the benchmark batch")
        self.tokens: List[int] = [0] * len(prompts)
        out = torch.empty(1, dtype=torch.int32, device=engine.device)
        for i, (rid, prompt) in enumerate(zip(self.ids, prompts)):
            at = 0
            while at < len(prompt):
                n = min(prefill_budget, len(prompt) - at)
                last = at + n == len(prompt)
                logits = engine.step([StepEntry(rid, prompt[at:at + n], [n - 1] if last else [])])
                at += n
            ops.argmax_rows(logits, out)
            self.tokens[i] = int(out.item())
        self.picked = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
        self.graph = None
        if use_graph and graph_capable(engine):
            greedy = GenerationConfig(max_new_tokens=max_steps, temperature=0.0)
            self.lengths = [cache.length(rid) for rid in self.ids]
            for rid, n in zip(self.ids, self.lengths):
                if not cache.reserve(rid, n + 1):
                    raise RuntimeError("no pages for the benchmark batch")
            pool = DecodeGraphPool(engine)
            self.graph = pool.get(self.ids, headroom_tokens=max_steps)
            state = (self.tokens, self.lengths, [greedy] * len(self.ids), [1] * len(self.ids))
            self.graph.load(self.ids, *state)
            pool.ensure_captured(self.graph)
            self.graph.load(self.ids, *state)

    def step(self) -> None:
        if self.graph is None:
            logits = self.engine.step([StepEntry(rid, [t], [0]) for rid, t in zip(self.ids, self.tokens)])
            ops.argmax_rows(logits, self.picked)
            self.tokens = self.picked.tolist()
            return
        cache = self.engine.cache
        for i, rid in enumerate(self.ids):                       # a page for the token this step stores
            if not cache.reserve(rid, self.lengths[i] + 1):
                raise RuntimeError("the benchmark batch ran out of pages")
        self.graph.refresh_tables()
        self.graph.replay()
        for i, rid in enumerate(self.ids):
            self.lengths[i] += 1
            cache.commit(rid, self.lengths[i])

    def context_length(self) -> int:
        return max(self.engine.cache.length(rid) for rid in self.ids)

    def close(self) -> None:
        for rid in self.ids:
            self.engine.cache.release(rid)


def count_launches(session: DecodeSession) -> int:
    """Kernels of this library launched by one decode step."""
    if session.graph is not None:
        return session.graph.launches_per_replay
    before = LaunchCounter.own
    session.step()
    return LaunchCounter.own - before
