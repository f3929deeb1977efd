"""GPT-2 (``GPT2LMHeadModel``) expressed as a :class:`ModelSpec`, and its random
initialisation.

Structure and tensor names follow the reference's loader
(heteroserve/model/weights.py:61-100): ``wte.weight``, ``wpe.weight``, per layer
``h.{i}.ln_1``, ``h.{i}.attn.c_attn`` (fused q|k|v, stored [in, out]),
``h.{i}.attn.c_proj``, ``h.{i}.ln_2``, ``h.{i}.mlp.c_fc``, ``h.{i}.mlp.c_proj``, then
``ln_f``; the head is the token table (weights.py:40-43).  Prefixes ``transformer.``
and ``model.`` are dropped (weights.py:54-58).
"""

from __future__ import annotations

import math

import torch

from ..config.model_config import GPT2_ACTIVATIONS, Architecture, GPT2Config, register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: GPT2Config) -> ModelSpec:
    E, H, D, I = cfg.n_embd, cfg.n_head, cfg.head_dim, cfg.inner_dim
    act = GPT2_ACTIVATIONS[cfg.activation_function]
    layers = []
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        layers.append(LayerSpec(
            arrangement="pre_norm",
            norm1=PartSpec("layernorm", dict(width=E, eps=cfg.layer_norm_epsilon,
                                             weight=p + "ln_1.weight", bias=p + "ln_1.bias")),
            mixer=PartSpec("causal_attention", dict(
                width=E, n_heads=H, head_dim=D, scale=cfg.attention_scale(i),
                qkv_weight=p + "attn.c_attn.weight", qkv_bias=p + "attn.c_attn.bias",
                out_weight=p + "attn.c_proj.weight", out_bias=p + "attn.c_proj.bias",
                stored_in_out=True)),
            norm2=PartSpec("layernorm", dict(width=E, eps=cfg.layer_norm_epsilon,
                                             weight=p + "ln_2.weight", bias=p + "ln_2.bias")),
            feed_forward=PartSpec("dense", dict(
                width=E, inner=I, activation=act,
                in_weight=p + "mlp.c_fc.weight", in_bias=p + "mlp.c_fc.bias",
                out_weight=p + "mlp.c_proj.weight", out_bias=p + "mlp.c_proj.bias",
                stored_in_out=True)),
        ))
    head_weight = "wte.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    ignore = [r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"]
    if cfg.tie_word_embeddings:
        ignore.append(r"lm_head\.weight")
    return ModelSpec(
        name="GPT2LMHeadModel", vocab_size=cfg.vocab_size, width=E,
        max_positions=cfg.n_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab_size, width=E,
                                               table="wte.weight")),
        position=PartSpec("learned", dict(max_positions=cfg.n_positions, width=E,
                                          table="wpe.weight")),
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(cfg.n_layer)),
        final_norm=PartSpec("layernorm", dict(width=E, eps=cfg.layer_norm_epsilon,
                                              weight="ln_f.weight", bias="ln_f.bias")),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab_size, width=E, weight=head_weight)),
        eos_token_id=cfg.eos_token_id,
        strip_prefixes=("transformer.", "model."),
        ignore_tensors=tuple(ignore),
    )


def init_weights(cfg: GPT2Config, seed: int) -> dict[str, torch.Tensor]:
    """Seeded random float32 weights under the checkpoint's own names.

    Tables and linear weights ~ N(0, 0.02); both ``c_proj`` weights
    ~ N(0, 0.02 / sqrt(2 * n_layer)); biases ~ N(0, 0.01); LayerNorm weight
    1 + N(0, 0.02) and bias N(0, 0.02).  (The reference's ``synthetic_gpt2`` draws only the
    matrices and leaves biases 0 and norms at identity, heteroserve/model/weights.py:103-142;
    non-trivial biases and norms make a mistake in either visible.)

    One CPU generator seeded with ``seed`` is drawn from in this fixed order:
    wte, wpe, then for each layer ln_1.weight, ln_1.bias, c_attn.weight, c_attn.bias,
    attn.c_proj.weight, attn.c_proj.bias, ln_2.weight, ln_2.bias, c_fc.weight, c_fc.bias,
    mlp.c_proj.weight, mlp.c_proj.bias, then ln_f.weight, ln_f.bias (and lm_head.weight if
    the head is untied)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    E, I = cfg.n_embd, cfg.inner_dim
    proj_std = 0.02 / math.sqrt(2.0 * cfg.n_layer)

    def normal(shape, std, mean=0.0):
        return torch.randn(shape, generator=gen, dtype=torch.float32) * std + mean

    w: dict[str, torch.Tensor] = {}
    w["wte.weight"] = normal((cfg.vocab_size, E), 0.02)
    w["wpe.weight"] = normal((cfg.n_positions, E), 0.02)
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        w[p + "ln_1.weight"] = normal((E,), 0.02, 1.0)
        w[p + "ln_1.bias"] = normal((E,), 0.02)
        w[p + "attn.c_attn.weight"] = normal((E, 3 * E), 0.02)
        w[p + "attn.c_attn.bias"] = normal((3 * E,), 0.01)
        w[p + "attn.c_proj.weight"] = normal((E, E), proj_std)
        w[p + "attn.c_proj.bias"] = normal((E,), 0.01)
        w[p + "ln_2.weight"] = normal((E,), 0.02, 1.0)
        w[p + "ln_2.bias"] = normal((E,), 0.02)
        w[p + "mlp.c_fc.weight"] = normal((E, I), 0.02)
        w[p + "mlp.c_fc.bias"] = normal((I,), 0.01)
        w[p + "mlp.c_proj.weight"] = normal((I, E), proj_std)
        w[p + "mlp.c_proj.bias"] = normal((E,), 0.01)
    w["ln_f.weight"] = normal((E,), 0.02, 1.0)
    w["ln_f.bias"] = normal((E,), 0.02)
    if not cfg.tie_word_embeddings:
        w["lm_head.weight"] = normal((cfg.vocab_size, E), 0.02)
    return w


GPT2 = Architecture(name="GPT2LMHeadModel", config_cls=GPT2Config, build_spec=build_spec,
                    init_weights=init_weights, model_types=("gpt2",))
register_architecture(GPT2, replace=True)
