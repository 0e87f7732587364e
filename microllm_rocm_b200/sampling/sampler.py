"""Token selection for a batch of logits rows: one kernel launch, one small copy back.

Greedy rows and sampled rows share the launch (the kernel takes the greedy branch per
row).  The draw of a sampled row is a pure function of (seed, how many tokens the request
has drawn so far), so a request gets the same tokens whatever it is batched with and
however often it was preempted and recomputed.  See csrc/sampling.cu for the definition
and its relation to the reference's sampler (src/inference/generator.cpp:36-69).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from .config import GenerationConfig


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, configs: Sequence[GenerationConfig], draws: Sequence[int]) -> List[int]:
        """logits [R, V] fp32 on the device; configs/draws one per row.  Returns R token ids
        on the host (-1 for a row with a non-finite logit)."""
        return self.sample_device(logits, configs, draws).tolist()

    def sample_device(self, logits: torch.Tensor, configs: Sequence[GenerationConfig], draws: Sequence[int]) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        return self.sample_into(logits, configs, draws, out)

    def sample_into(self, logits: torch.Tensor, configs: Sequence[GenerationConfig], draws: Sequence[int],
                    out: torch.Tensor) -> torch.Tensor:
        R = logits.shape[0]
        if R != len(configs) or R != len(draws) or out.shape[0] != R:
            raise ValueError("one config, one draw index and one output slot per logits row")
        if R == 0:
            return out
        if all(c.greedy for c in configs):
            ops.argmax_rows(logits, out)
            return out
        # (uploads through pinned memory: they must not wait for what the GPU is still running)
        temperature = ops.upload([0.0 if c.greedy else c.temperature for c in configs], "float32", self.device)
        top_k = ops.upload([c.top_k for c in configs], "int32", self.device)
        seed = ops.upload([c.seed for c in configs], "int64", self.device)
        draw = ops.upload(list(draws), "int64", self.device)
        ops.sample_rows(logits, temperature, top_k, seed, draw, out)
        return out
