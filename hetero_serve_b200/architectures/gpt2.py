"""GPT-2 (``GPT2LMHeadModel``): its typed configuration, its :class:`ModelSpec`, its
random initialisation and its named configurations.  Everything the framework knows about
this architecture is in this file; another architecture is another file like it.

Structure and tensor names follow the reference's loader
(heteroserve/model/weights.py:61-100): ``wte.weight``, ``wpe.weight``, per layer
``h.{i}.ln_1``, ``h.{i}.attn.c_attn`` (fused q|k|v, stored [in, out]),
``h.{i}.attn.c_proj``, ``h.{i}.ln_2``, ``h.{i}.mlp.c_fc``, ``h.{i}.mlp.c_proj``, then
``ln_f``; the head is the token table (weights.py:40-43).  Prefixes ``transformer.``
and ``model.`` are dropped (weights.py:54-58).
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass, fields
from typing import Any, Mapping

import torch

from ..config.model_config import (Architecture, ConfigError, flag, need, positive_int,
                                   register_architecture)
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


GPT2_ACTIVATIONS = {
    # name in config.json -> activation kind the feed-forward part understands
    "gelu_new": "gelu_tanh",
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu": "gelu_erf",
}


@dataclass(frozen=True)
class GPT2Config:
    """The GPT-2 dense decoder (``GPT2LMHeadModel``) as its config.json spells it.

    The reference reads ``n_layer/n_head/n_embd/vocab_size/n_ctx/layer_norm_epsilon``
    (heteroserve/config.py:59-70) and fixes the rest in code (4x inner width,
    tanh-GELU, 1/sqrt(head_dim) scale: heteroserve/model/weights.py:129-130,
    heteroserve/model/torch_engine.py:47,78).  Here those are configuration too.
    """

    n_layer: int
    n_embd: int
    n_head: int
    vocab_size: int
    n_positions: int
    n_inner: int | None = None                  # None → 4 * n_embd
    layer_norm_epsilon: float = 1e-5            # reference default, config.py:69
    activation_function: str = "gelu_new"
    scale_attn_weights: bool = True             # scores * 1/sqrt(head_dim)
    scale_attn_by_inverse_layer_idx: bool = False   # additionally / (layer_idx + 1)
    tie_word_embeddings: bool = True
    eos_token_id: int | None = None
    architectures: tuple[str, ...] = ("GPT2LMHeadModel",)
    model_type: str = "gpt2"

    # -- derived ---------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    def kv_bytes_per_token(self, itemsize: int) -> int:
        """Bytes of K and V one token occupies over all layers (config.py:54-56)."""
        return 2 * self.n_layer * self.n_head * self.head_dim * itemsize

    def attention_scale(self, layer_idx: int) -> float:
        """Score multiplier of one layer, formed once in float64.

        ``1/sqrt(head_dim)`` as in heteroserve/model/torch_engine.py:47 when
        ``scale_attn_weights``; divided by ``layer_idx + 1`` (zero-based index)
        when ``scale_attn_by_inverse_layer_idx``.  The kernels and the plain
        implementation both round this one number to 32-bit and apply it as a
        single multiply after the dot product.
        """
        s = 1.0 / math.sqrt(self.head_dim) if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            s = s / float(layer_idx + 1)
        return s

    def num_parameters(self) -> int:
        e, i, v, p = self.n_embd, self.inner_dim, self.vocab_size, self.n_positions
        per_layer = 4 * e + (e * 3 * e + 3 * e) + (e * e + e) + (e * i + i) + (i * e + e)
        n = v * e + p * e + self.n_layer * per_layer + 2 * e
        if not self.tie_word_embeddings:
            n += v * e
        return n

    # -- io ---------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "GPT2Config":
        n_layer = positive_int("n_layer", need(raw, "n_layer"))
        n_embd = positive_int("n_embd", need(raw, "n_embd"))
        n_head = positive_int("n_head", need(raw, "n_head"))
        vocab = positive_int("vocab_size", need(raw, "vocab_size"))
        # the reference spells the table length n_ctx (config.py:68)
        n_pos = positive_int("n_positions", need(raw, "n_positions", "n_ctx"))
        if "n_positions" in raw and "n_ctx" in raw and raw["n_ctx"] is not None \
                and raw["n_positions"] is not None and raw["n_ctx"] != raw["n_positions"]:
            raise ConfigError(
                f"n_positions ({raw['n_positions']}) and n_ctx ({raw['n_ctx']}) disagree")
        if n_embd % n_head:
            raise ConfigError(f"n_embd ({n_embd}) is not a multiple of n_head ({n_head})")
        n_inner = raw.get("n_inner")
        if n_inner is not None:
            n_inner = positive_int("n_inner", n_inner)
        eps = raw.get("layer_norm_epsilon", 1e-5)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not eps > 0:
            raise ConfigError(f"layer_norm_epsilon must be a positive number, got {eps!r}")
        act = raw.get("activation_function", "gelu_new")
        if act not in GPT2_ACTIVATIONS:
            raise ConfigError(
                f"activation_function {act!r} is not supported; "
                f"known: {sorted(GPT2_ACTIVATIONS)}")
        eos = raw.get("eos_token_id")
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int)):
            raise ConfigError(f"eos_token_id must be an integer, got {eos!r}")
        archs = raw.get("architectures") or ("GPT2LMHeadModel",)
        return cls(
            n_layer=n_layer, n_embd=n_embd, n_head=n_head, vocab_size=vocab,
            n_positions=n_pos, n_inner=n_inner, layer_norm_epsilon=float(eps),
            activation_function=act,
            scale_attn_weights=flag("scale_attn_weights", raw.get("scale_attn_weights", True)),
            scale_attn_by_inverse_layer_idx=flag(
                "scale_attn_by_inverse_layer_idx",
                raw.get("scale_attn_by_inverse_layer_idx", False)),
            tie_word_embeddings=flag("tie_word_embeddings",
                                      raw.get("tie_word_embeddings", True)),
            eos_token_id=eos,
            architectures=tuple(archs),
            model_type=raw.get("model_type", "gpt2"),
        )

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def replace(self, **kw) -> "GPT2Config":
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d.update(kw)
        return GPT2Config(**d)


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


# ``gpt2`` is the reference's default ``ModelConfig()`` (heteroserve/config.py:22-33); ``tiny``
# is its ``ModelConfig.tiny()`` (config.py:72-83); the others are the sizes the benchmark and
# the tests name.
_BASE = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
         "tie_word_embeddings": True, "eos_token_id": 50256}

PRESETS: dict[str, dict] = {  # config.json dictionaries
    "tiny-a": dict(_BASE, n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512,
                   n_positions=128, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                   scale_attn_by_inverse_layer_idx=False, eos_token_id=511),
    "tiny-b": dict(_BASE, n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000,
                   n_positions=256, layer_norm_epsilon=1e-6, activation_function="gelu",
                   scale_attn_by_inverse_layer_idx=True, eos_token_id=999),
    "tiny": dict(_BASE, n_layer=4, n_embd=256, n_head=4, n_inner=None, vocab_size=50257,
                 n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2": dict(_BASE, n_layer=12, n_embd=768, n_head=12, n_inner=None, vocab_size=50257,
                 n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2-medium": dict(_BASE, n_layer=24, n_embd=1024, n_head=16, n_inner=4096,
                        vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                        activation_function="gelu_new"),
    "gpt2-large": dict(_BASE, n_layer=36, n_embd=1280, n_head=20, n_inner=5120,
                       vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                       activation_function="gelu_new"),
    "gpt2-xl": dict(_BASE, n_layer=48, n_embd=1600, n_head=25, n_inner=6400,
                    vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                    activation_function="gelu_new"),
}
_ALIASES = {"tinya": "tiny-a", "tinyb": "tiny-b", "medium": "gpt2-medium",
            "large": "gpt2-large", "xl": "gpt2-xl"}

GPT2 = Architecture(name="GPT2LMHeadModel", config_cls=GPT2Config, build_spec=build_spec,
                    init_weights=init_weights, model_types=("gpt2",), presets=PRESETS,
                    preset_aliases=_ALIASES)
register_architecture(GPT2, replace=True)
