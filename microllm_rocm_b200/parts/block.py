"""Pre-norm residual block:  x += mixer(norm1(x));  x += feed_forward(norm2(x)).
Each residual add is fused into the norm that follows it (the reference does so on its
decode path only: src/model/model.cpp:862-870 `add_rms_norm`), so the block passes the
residual stream on together with a delta that has not been added yet."""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, FeedForward, Mixer, Norm, Runtime, StepContext, register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, params: dict, rt: Runtime, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm,
                 feed_forward: FeedForward):
        self.rt = rt
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward

    def replay_key(self):
        keys = [p.replay_key() for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)]
        return None if any(k is None for k in keys) else ("pre_norm_residual", self.rt.dtype, *keys)

    def own_tensors(self):
        return [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) for t in p.own_tensors()]

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache):
        normed = ctx.buffer("block.normed", tuple(residual.shape), self.rt.dtype)
        if delta is None:
            self.mixer_norm.forward(residual, normed)
        else:
            self.mixer_norm.add_forward(residual, delta, normed)
        mixed = self.mixer.forward(normed, ctx, cache)
        normed2 = ctx.buffer("block.normed2", tuple(residual.shape), self.rt.dtype)
        self.ffn_norm.add_forward(residual, mixed, normed2)
        return residual, self.feed_forward.forward(normed2, ctx)
