"""Qwen2 dense decoder as data: which parts, with which sizes, in which order.

token embedding -> L x [RMSNorm -> GQA attention (QKV bias, split-half RoPE) -> residual
-> RMSNorm -> SwiGLU MLP -> residual] -> RMSNorm -> LM head (tied or not).
Structure and tensor names as in the reference's model and name mapping
(src/model/model.cpp:820-908 block, :1928-1982 `qwen_style_weight_mapping`).

This file only describes; the parts it names live in `parts/` and know nothing of it.
"""
from __future__ import annotations

from ..config.qwen2 import ARCHITECTURE, PRESETS, Qwen2Config
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec


def build_spec(cfg: Qwen2Config) -> ModelSpec:
    cfg.validate()
    h, d = cfg.hidden_size, cfg.head_size
    position = PartSpec("rotary", dict(head_dim=d, rotary_dim=d, theta=float(cfg.rope_theta),
                                       layout="split_half"))
    layers = []
    for l in range(cfg.num_hidden_layers):
        norm = lambda sub: PartSpec("rmsnorm", dict(prefix=sub, size=h, eps=float(cfg.rms_norm_eps)))
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}.",
            block=PartSpec("pre_norm_residual"),
            mixer_norm=norm("input_layernorm."),
            mixer=PartSpec("attention", dict(
                prefix="self_attn.", hidden_size=h, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=d,
                qkv_bias=True,                    # fixed for qwen2 (huggingface.cpp:175)
                out_bias=False,                   # o_proj never has one (model.cpp:400)
                window=cfg.layer_window(l))),
            ffn_norm=norm("post_attention_layernorm."),
            feed_forward=PartSpec("swiglu", dict(prefix="mlp.", hidden_size=h,
                                                 intermediate_size=cfg.intermediate_size)),
        ))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=h, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(name="model.embed_tokens.weight",
                                                   vocab_size=cfg.vocab_size, hidden_size=h)),
        position=position,
        layers=layers,
        order=[RunSpec(layer=l) for l in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(prefix="model.norm.", size=h, eps=float(cfg.rms_norm_eps))),
        head=PartSpec("lm_head", dict(name="lm_head.weight", vocab_size=cfg.vocab_size, hidden_size=h,
                                      tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None)),
    )
    spec.validate()
    return spec


register_architecture(Architecture(name=ARCHITECTURE, config_class=Qwen2Config, build_spec=build_spec,
                                   model_types=("qwen2",), presets=PRESETS), replace=True)
