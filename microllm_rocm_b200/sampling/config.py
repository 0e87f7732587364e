"""Generation options, with the reference's names, meanings and defaults
(include/microllm/inference/generator.h:11-23)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Tuple


@dataclass(frozen=True)
class GenerationConfig:
    max_new_tokens: int = 32          # 0 returns at once with nothing generated
    temperature: float = 1.0          # 0 means greedy argmax; otherwise logits are divided by it
    top_k: int = 0                    # 0: whole vocabulary; 1: greedy; else the k largest logits
    seed: int = 1                     # one stream of draws per request
    stop_tokens: Tuple[int, ...] = field(default_factory=tuple)   # generation stops after appending one

    def __post_init__(self):
        object.__setattr__(self, "stop_tokens", tuple(int(t) for t in self.stop_tokens))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    def validate(self, vocab_size: int) -> None:
        """The reference's checks (src/inference/generator.cpp:15-28, 38-45;
        src/inference/scheduler.cpp:32-63)."""
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be non-negative")
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ValueError("sampling temperature must be finite and non-negative")
        if self.top_k < 0 or self.top_k > vocab_size:
            raise ValueError("top_k is outside the vocabulary")
        if len(set(self.stop_tokens)) != len(self.stop_tokens):
            raise ValueError("generation stop tokens must be unique")
        for t in self.stop_tokens:
            if not 0 <= t < vocab_size:
                raise ValueError("generation stop token is outside the vocabulary")
        if not 0 <= self.seed < 2 ** 63:
            raise ValueError("seed must fit in 63 bits")


SamplingParams = GenerationConfig
