"""GPT-2 (`GPT2LMHeadModel`) described as a ModelSpec.

Structure: src/models/gpt2_small.sandy.go:1-59 of the reference (token + position
embedding, pre-LayerNorm blocks of fused-QKV causal attention and a gelu MLP, final
LayerNorm, output head tied to the token table).  Tensor names are those of the HF
checkpoint the reference converts from (scripts/run_gpt2.py:160-189): `wte.weight`,
`wpe.weight`, `h.N.ln_1.*`, `h.N.attn.c_attn.*`, `h.N.attn.c_proj.*`, `h.N.ln_2.*`,
`h.N.mlp.c_fc.*`, `h.N.mlp.c_proj.*`, `ln_f.*`, with or without a `transformer.` prefix.
Linear weights are in Conv1D layout [in, out] and are used as stored.

Every number below comes from the GPT2Config.
"""
from __future__ import annotations

import math

from ..config.gpt2 import GPT2Config
from ..registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def describe_gpt2(cfg: GPT2Config) -> ModelSpec:
    E, H, D = cfg.n_embd, cfg.n_head, cfg.head_dim
    layers = []
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        # scale_attn_weights: scores * 1/sqrt(D); scale_attn_by_inverse_layer_idx: also / (i+1).
        # The reference's attention takes this as its `scale` attribute
        # (src/core/TensorCalc.cpp:1236-1237: default 1/sqrt(D) when none is given).
        scale = 1.0
        if cfg.scale_attn_weights:
            scale /= math.sqrt(D)
        if cfg.scale_attn_by_inverse_layer_idx:
            scale /= float(i + 1)
        norm = lambda name: PartSpec("layernorm", {"width": E, "eps": cfg.layer_norm_epsilon, "bias": True},
                                     {"weight": p + name + ".weight", "bias": p + name + ".bias"})
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=PartSpec("causal_attention",
                           {"width": E, "n_heads": H, "n_kv_heads": H, "head_dim": D, "scale": scale,
                            "window": None, "bias": True, "weight_layout": "in_out"},
                           {"qkv.weight": p + "attn.c_attn.weight", "qkv.bias": p + "attn.c_attn.bias",
                            "out.weight": p + "attn.c_proj.weight", "out.bias": p + "attn.c_proj.bias"}),
            feed_forward=PartSpec("dense_mlp",
                                  {"width": E, "inner": cfg.inner_dim, "activation": cfg.activation_function,
                                   "bias": True, "weight_layout": "in_out"},
                                  {"up.weight": p + "mlp.c_fc.weight", "up.bias": p + "mlp.c_fc.bias",
                                   "down.weight": p + "mlp.c_proj.weight", "down.bias": p + "mlp.c_proj.bias"}),
            norms={"mixer": norm("ln_1"), "feed_forward": norm("ln_2")},
        ))
    head_tensors = {} if cfg.tie_word_embeddings else {"weight": "lm_head.weight"}
    ignored = [r"^h\.\d+\.attn\.(bias|masked_bias)$"]   # stored causal-mask buffers of old checkpoints
    if cfg.tie_word_embeddings:
        ignored.append(r"^lm_head\.weight$")            # a stored copy of the tied table
    return ModelSpec(
        architecture=cfg.architecture,
        width=E,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.n_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": E}, {"weight": "wte.weight"}),
        position=PartSpec("learned_absolute", {"width": E, "max_positions": cfg.n_positions},
                          {"weight": "wpe.weight"}),
        layers=layers,
        schedule=[LayerCall(layer=i, cache=i, write_cache=True) for i in range(cfg.n_layer)],
        final_norm=PartSpec("layernorm", {"width": E, "eps": cfg.layer_norm_epsilon, "bias": True},
                            {"weight": "ln_f.weight", "bias": "ln_f.bias"}),
        head=PartSpec("output_head", {"vocab_size": cfg.vocab_size, "width": E, "tied": cfg.tie_word_embeddings},
                      head_tensors),
        name_prefixes=("", "transformer."),
        ignored_tensors=tuple(ignored),
        eos_token_id=cfg.eos_token_id,
    )


register_architecture(GPT2Config.architecture, GPT2Config, describe_gpt2)
