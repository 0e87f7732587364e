"""Grouped-query attention over the paged cache.

  q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv      one fused product (the reference runs
                                                       three: src/model/model.cpp:457-476)
  q, k rotated by the position encoding's table; k, v stored into this run's pages
  head h attends with kv head h // (NH/NKV) over keys lo..pos, scale 1/sqrt(D) after the dot
  out = concat_heads(o) Wo^T

All sizes are parameters; `window` (keys visible, itself included) is per layer and may be
None.  The part never learns which layer or model it belongs to.  Formulas:
src/model/model.cpp:447-523 (prefill), :525-603 (decode); scale at :513-514.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import attention as attention_kernels
from ..kernels import gemm_bf16, ops
from ..kernels.linear import linear
from .base import Mixer, PagedKVNeed, PagedKVView, PositionEncoding, Runtime, StepContext, WeightSpec, register_mixer


ROPE_TABLE_MIN_TOKENS = 64          # from here on a step-wide table of sines and cosines pays


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.qkv_bias = bool(params.get("qkv_bias", False))
        self.out_bias = bool(params.get("out_bias", False))
        self.window = params.get("window")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(float(self.d))))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        attention_kernels.check_head_dim(self.d)
        self.rt = rt
        self.rotary = position.rotary_table(self.d) if position is not None else None
        if self.rotary is None:        # no rotation: an empty table makes the kernel pass q/k through
            self._no_rot = torch.zeros(0, dtype=torch.float32, device=rt.device)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    # --- declarations -----------------------------------------------------------------
    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, kv = self.nh * self.d, self.nkv * self.d
        specs = {"q_proj.weight": WeightSpec((q, self.hidden)), "k_proj.weight": WeightSpec((kv, self.hidden)),
                 "v_proj.weight": WeightSpec((kv, self.hidden)), "o_proj.weight": WeightSpec((self.hidden, q))}
        if self.qkv_bias:
            specs.update({"q_proj.bias": WeightSpec((q,), role="vector"), "k_proj.bias": WeightSpec((kv,), role="vector"),
                          "v_proj.bias": WeightSpec((kv,), role="vector")})
        if self.out_bias:
            specs["o_proj.bias"] = WeightSpec((self.hidden,), role="vector")
        return specs

    def fused_tensors(self):
        q, kv = self.nh * self.d, self.nkv * self.d
        fused = {"qkv_proj.weight": (WeightSpec((q + 2 * kv, self.hidden)),
                                     [("q_proj.weight", 0), ("k_proj.weight", q), ("v_proj.weight", q + kv)])}
        if self.qkv_bias:
            fused["qkv_proj.bias"] = (WeightSpec((q + 2 * kv,), role="vector"),
                                      [("q_proj.bias", 0), ("k_proj.bias", q), ("v_proj.bias", q + kv)])
        return fused

    def bind(self, tensors):
        # the loader hands over the fused tensors; a caller with the checkpoint's pieces gets them joined here
        if "qkv_proj.weight" in tensors:
            self.w_qkv = tensors["qkv_proj.weight"]
            self.b_qkv = tensors.get("qkv_proj.bias") if self.qkv_bias else None
        else:
            self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], 0).contiguous()
            if self.qkv_bias:
                self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], 0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def kernel_sources(self):
        if self.rt.is_fp32:
            return []
        return (gemm_bf16.sources(engine_only=True) + attention_kernels.mma_sources(self.d)
                + attention_kernels.tc_sources(self.d))

    def replay_key(self):
        if self.out_bias:
            return None                  # a bias on the output projection is added by a tensor-framework operation
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None                  # the library product would go through the tensor framework
        rotary = None if self.rotary is None else (self.rotary.inv_freq.data_ptr(), self.rotary.rotary_dim, self.rotary.interleaved)
        return ("attention", self.hidden, self.nh, self.nkv, self.d, self.qkv_bias, self.window, self.scale, rotary)

    def own_tensors(self):
        return [self.w_qkv, self.b_qkv, self.w_o]

    # --- launch plans frozen into a captured decode step ----------------------------------
    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        from ..kernels.device import sm_count
        return attention_kernels.decode_plan_stale(ctx, max_seq_len, sm_count(self.rt.device))

    def forget_plans(self, ctx: StepContext) -> None:
        attention_kernels.forget_plans(ctx)

    def plan_group(self):
        return ("attention", self.rt.device)          # the kernels' plans are kept per (group size, kv heads), for all layers

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        T = x.shape[0]
        q = ctx.buffer("attention.q", (T, self.nh * self.d), self.rt.dtype)
        inv_freq, rot, inter = ((self.rotary.inv_freq, self.rotary.rotary_dim, self.rotary.interleaved)
                                if self.rotary is not None else (self._no_rot, 0, False))
        pages = cache.pages if cache.writable else None
        if (x.dtype == torch.bfloat16 and gemm_bf16.gemv_preferred(x, self.w_qkv)
                and gemm_bf16.gemv_fused_supported(x, self.w_qkv) and self.d % 16 == 0
                and (rot == 0 or (rot == self.d and not inter))):
            # a few tokens: projection, bias, rotation and the cache store in one weight-streaming kernel
            gemm_bf16.gemv_qkv_rope(x, self.w_qkv, self.b_qkv, ctx.positions, ctx.token_seq, cache.block_table,
                                    inv_freq if rot else None, q, pages, self.nh, self.nkv, self.d, ctx.error_flag)
        else:
            qkv = linear(x, self.w_qkv, None, torch.float32, partials_ok=True,    # [T, (NH+2NKV)*D] f32, or its partial sums
                         alloc=lambda shape, dtype: ctx.buffer("attention.qkv", shape, dtype), error_flag=ctx.error_flag)
            cos_sin = None
            if rot and T >= ROPE_TABLE_MIN_TOKENS and x.dtype == torch.bfloat16:
                # a prompt portion: the step's sines and cosines are made once and serve every layer and head
                # (a result of this step's positions: it lives in step_values, which every forward starts empty,
                # so a context that outlives its step -- a captured decode step -- never reads old angles)
                key = ("rope_table", id(self.rotary))
                cos_sin = ctx.step_values.get(key)
                if cos_sin is None:
                    table = ctx.buffer("attention.rope_table", (T, rot // 2, 2), torch.float32)
                    cos_sin = ctx.step_values[key] = ops.rope_table(ctx.positions, inv_freq, out=table)
            ops.rope_kv_write(qkv, self.b_qkv, ctx.positions, ctx.token_seq, cache.block_table, inv_freq, rot, inter,
                              q, pages, self.nh, self.nkv, self.d, ctx.error_flag, cos_sin)
        o = ctx.buffer("attention.o", (T, self.nh * self.d), self.rt.dtype)
        attention_kernels.paged_attention(q, cache.pages, o, ctx, cache.block_table, self.nh, self.nkv, self.d,
                                          self.scale, self.window,
                                          beside_mma_products=x.dtype == torch.bfloat16 and gemm_bf16.gemv_preferred(x, self.w_o))
        return linear(o, self.w_o, self.b_o, torch.float32, partials_ok=True, error_flag=ctx.error_flag,      # [T, H] f32, or its partial sums
                      alloc=lambda shape, dtype: ctx.buffer("attention.out", shape, dtype))
