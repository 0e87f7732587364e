"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ), no biases
(reference: src/model/model.cpp:757-794; activation src/ops/ops.cpp:760-785).
Gate and up are one fused product (gate rows first, then up rows)."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import gemm_bf16, ops
from ..kernels.linear import linear
from .base import FeedForward, Runtime, StepContext, WeightSpec, register_feed_forward, scratch


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.rt = rt
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"gate_proj.weight": WeightSpec((self.inter, self.hidden)),
                "up_proj.weight": WeightSpec((self.inter, self.hidden)),
                "down_proj.weight": WeightSpec((self.hidden, self.inter))}

    def kernel_sources(self):
        return [] if self.rt.is_fp32 else gemm_bf16.sources(engine_only=True)

    def fused_tensors(self):
        return {"gate_up_proj.weight": (WeightSpec((2 * self.inter, self.hidden)),
                                        [("gate_proj.weight", 0), ("up_proj.weight", self.inter)])}

    def bind(self, tensors):
        if "gate_up_proj.weight" in tensors:             # from the loader: already fused, gate rows then up rows
            self.w_gate_up = tensors["gate_up_proj.weight"]
        else:
            self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], 0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None                  # the library product would go through the tensor framework
        return ("swiglu", self.hidden, self.inter)

    def own_tensors(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        # fp32 path: everything f32.  bf16 path: gate/up leave the product as bf16, the
        # activation is evaluated in fp32 and stored bf16, down returns fp32 at the residual
        # boundary -- the reference's policy for its bf16 feed-forward (src/ops/optimized.cpp:676-683).
        act = scratch(ctx, "swiglu.act", (x.shape[0], self.inter), self.rt.dtype, x.device)
        flag = ctx.error_flag if ctx is not None else None      # one flag covers the step: whoever reads it sees every kernel's
        if (x.dtype == torch.bfloat16 and x.shape[0] <= gemm_bf16.GEMV_SILU_MAX_TOKENS and gemm_bf16.gemv_preferred(x, self.w_gate_up)
                and gemm_bf16.gemv_fused_supported(x, self.w_gate_up)):
            # a few tokens: one weight-streaming kernel, the activation is its epilogue
            gemm_bf16.gemv_silu_mul(x, self.w_gate_up, act)
        elif x.dtype == torch.bfloat16 and gemm_bf16.gemv_preferred(x, self.w_gate_up):
            # more tokens, or a width too large for that kernel: fp32 partial sums, the activation adds them
            ops.silu_mul(gemm_bf16.gemv_partials(x, self.w_gate_up, alloc=lambda shape, dtype: scratch(
                ctx, "swiglu.gate_up_partials", shape, dtype, x.device)), act)
        elif gemm_bf16.stream_preferred(x, self.w_gate_up):
            # up to 128 tokens: the tcgen05 weight-streaming product, the activation is its epilogue
            gemm_bf16.stream_silu_mul(x, self.w_gate_up, act, error_flag=flag)
        elif x.dtype == torch.bfloat16 and x.shape[0] >= gemm_bf16.PAIR_MIN_TOKENS and gemm_bf16.supported(x, self.w_gate_up):
            # a prompt portion: the CTA-pair tcgen05 product with the activation in its epilogue
            gemm_bf16.gemm_pair(x, self.w_gate_up, act, dual_rows=self.inter, error_flag=flag)
        else:
            gate_up = linear(x, self.w_gate_up, None, self.rt.dtype,
                             alloc=lambda shape, dtype: scratch(ctx, "swiglu.gate_up", shape, dtype, x.device))
            ops.silu_mul(gate_up, act)
        return linear(act, self.w_down, None, torch.float32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: scratch(ctx, "swiglu.out", shape, dtype, x.device))
