"""A fixed batch of requests in steady decode, for measurement: prompts are prefilled in
portions, then every `step()` feeds each request the token it was given last and selects
the next one greedily.  Counted tokens equal forward passes, as in the reference's steady
decode accounting (apps/hf_infer.cpp:1464-1468)."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from ..kernels.build import LaunchCounter
from .step import Engine, StepEntry


class DecodeSession:
    def __init__(self, engine: Engine, prompts: Sequence[Sequence[int]], max_steps: int, prefill_budget: int = 2048):
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

    def step(self) -> None:
        logits = self.engine.step([StepEntry(rid, [t], [0]) for rid, t in zip(self.ids, self.tokens)])
        ops.argmax_rows(logits, self.picked)
        self.tokens = self.picked.tolist()

    def context_length(self) -> int:
        return max(self.engine.cache.length(rid) for rid in self.ids)

    def close(self) -> None:
        for rid in self.ids:
            self.engine.cache.release(rid)


def count_launches(session: DecodeSession) -> int:
    """Kernels of this library launched by one decode step."""
    before = LaunchCounter.own
    session.step()
    return LaunchCounter.own - before
