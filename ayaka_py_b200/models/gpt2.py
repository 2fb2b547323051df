"""GPT-2 as data: which parts, with which constants, bound to which tensors.

Layer order and formulas: ``models/gpt2.py:429-438`` (block), ``:364-372``
(attention), ``:400-403`` (MLP), ``:516-517`` (embedding), ``:530`` (ln_f);
tensor names and Conv1D layout ``:152-251``; name rules ``:54-61``.
"""

from __future__ import annotations

import math

from ..config.model import GPT2Config
from ..parts.base import Init, ModelSpec, PartSpec, RunStep, Source, pre_norm_layer
from ..registry import Architecture, register_architecture

# layers/activation.py:198-203
_ACTIVATION_KIND = {"gelu": "gelu_erf", "gelu_new": "gelu_tanh", "gelu_fast": "gelu_tanh",
                    "gelu_pytorch_tanh": "gelu_tanh", "quick_gelu": "quick_gelu"}


def gpt2_spec(config: GPT2Config) -> ModelSpec:
    d, inner, eps = config.n_embd, config.inner_size, config.layer_norm_epsilon
    matrix = Init(std=0.02)
    residual_proj = Init(std=0.02 / math.sqrt(2.0 * config.n_layer))
    bias = Init(std=0.01)
    gamma, beta = Init(std=0.05, mean=1.0), Init(std=0.02)

    def norm(prefix: str) -> PartSpec:
        return PartSpec("layernorm", {"width": d, "eps": eps},
                        {"weight": Source(prefix + ".weight", init=gamma),
                         "bias": Source(prefix + ".bias", init=beta)})

    layers = []
    for i in range(config.n_layer):
        p = f"transformer.h.{i}."
        mixer = PartSpec(
            "attention",
            {"width": d, "num_heads": config.n_head, "kv_heads": config.n_head,
             "head_dim": config.head_dim, "scale": config.attention_scale(i),
             "window": None, "bias": True},
            {"qkv_weight": Source(p + "attn.c_attn.weight", transposed=True, init=matrix),
             "qkv_bias": Source(p + "attn.c_attn.bias", init=bias),
             "out_weight": Source(p + "attn.c_proj.weight", transposed=True, init=residual_proj),
             "out_bias": Source(p + "attn.c_proj.bias", init=bias)})
        ffn = PartSpec(
            "mlp",
            {"width": d, "inner": inner, "activation": _ACTIVATION_KIND[config.activation_function],
             "bias": True},
            {"up_weight": Source(p + "mlp.c_fc.weight", transposed=True, init=matrix),
             "up_bias": Source(p + "mlp.c_fc.bias", init=bias),
             "down_weight": Source(p + "mlp.c_proj.weight", transposed=True, init=residual_proj),
             "down_bias": Source(p + "mlp.c_proj.bias", init=bias)})
        layers.append(pre_norm_layer(norm(p + "ln_1"), mixer, norm(p + "ln_2"), ffn))

    head_source = "transformer.wte.weight" if config.tie_word_embeddings else "lm_head.weight"
    return ModelSpec(
        vocab_size=config.vocab_size,
        hidden_size=d,
        max_positions=config.n_positions,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab_size, "width": d},
                           {"weight": Source("transformer.wte.weight", init=matrix)}),
        position=PartSpec("learned_positions", {"positions": config.n_positions, "width": d},
                          {"weight": Source("transformer.wpe.weight", init=matrix)}),
        layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(config.n_layer)),
        final_norm=norm("transformer.ln_f"),
        head=PartSpec("lm_head", {"vocab": config.vocab_size, "width": d},
                      {"weight": Source(head_source, init=matrix)}),
    )


def gpt2_normalize_name(name: str, config: GPT2Config) -> str | None:
    """Legacy mask buffers are ignored; names without ``transformer.`` get it;
    a shipped ``lm_head.weight`` is dropped when the head is tied."""
    if name.endswith(".attn.bias") or name.endswith(".attn.masked_bias"):
        return None
    if name == "lm_head.weight":
        return None if config.tie_word_embeddings else name
    if not name.startswith("transformer."):
        return "transformer." + name
    return name


register_architecture(Architecture(
    name="GPT2LMHeadModel", model_type="gpt2", config_class=GPT2Config,
    build_spec=gpt2_spec, normalize_name=gpt2_normalize_name))
