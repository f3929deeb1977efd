"""Typed model configurations and the architecture registry.

A model folder carries a ``config.json`` in the architecture's own vocabulary
(for GPT-2: ``n_layer``, ``n_embd``, ``n_head``, ``n_inner``, ``n_positions``,
``vocab_size``, ``layer_norm_epsilon``, ``activation_function``,
``scale_attn_by_inverse_layer_idx`` ...).  Each architecture registers

* a frozen dataclass that reads and validates those keys, and
* a builder that turns the typed configuration into a :class:`ModelSpec`
  (``hetero_serve_b200.parts.spec``): a purely declarative description of the
  layers, their parts and the order in which they run.

Nothing else in the framework looks at ``config.json``; every size and
constant reaches the kernels through the spec.

The typed-dataclass manner follows the reference's ``ModelConfig``
(heteroserve/config.py:21-70), which reads ``n_layer``, ``n_head``, ``n_embd``,
``vocab_size``, ``n_ctx`` and ``layer_norm_epsilon``; the reference has no
registry (it picks the model with a string compare, heteroserve/worker/worker.py:832).
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any, Callable, Mapping


class ConfigError(ValueError):
    """A config.json that is missing a key, or whose values do not fit together."""


# ---------------------------------------------------------------------------
# registry
# ---------------------------------------------------------------------------


@dataclass(frozen=True)
class Architecture:
    """What the framework knows about one architecture name."""

    name: str
    config_cls: type
    build_spec: Callable[[Any], Any]          # typed config -> ModelSpec
    init_weights: Callable[[Any, int], dict]  # (typed config, seed) -> {name: fp32 tensor}
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    """Add an architecture; ``architectures[0]`` of config.json selects it."""
    if arch.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    for mt in arch.model_types:
        _MODEL_TYPES[mt] = arch.name


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.pop(name, None)
    if arch is not None:
        for mt in arch.model_types:
            if _MODEL_TYPES.get(mt) == name:
                del _MODEL_TYPES[mt]


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {registered_architectures()}"
        ) from None


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    """Pick the architecture a raw config.json dictionary names."""
    archs = raw.get("architectures")
    if archs:
        if not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
            raise ConfigError(f"'architectures' must be a list of names, got {archs!r}")
        return get_architecture(archs[0])
    mt = raw.get("model_type")
    if mt in _MODEL_TYPES:
        return _ARCHITECTURES[_MODEL_TYPES[mt]]
    raise ConfigError(
        "config.json names no known architecture: needs 'architectures': [name] "
        f"(or a known 'model_type'); registered: {registered_architectures()}"
    )


def load_model_config(model_dir: str | Path):
    """Read ``<model_dir>/config.json`` → ``(Architecture, typed config)``."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {model_dir}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    arch = architecture_of(raw)
    return arch, arch.config_cls.from_dict(raw)


# ---------------------------------------------------------------------------
# helpers for typed configs
# ---------------------------------------------------------------------------


def _need(raw: Mapping[str, Any], key: str, *alts: str):
    for k in (key, *alts):
        if k in raw and raw[k] is not None:
            return raw[k]
    names = " or ".join(repr(k) for k in (key, *alts))
    raise ConfigError(f"config.json is missing {names}")


def _pos_int(name: str, v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {v!r}")
    return v


def _flag(name: str, v: Any) -> bool:
    if not isinstance(v, bool):
        raise ConfigError(f"{name} must be true or false, got {v!r}")
    return v


# ---------------------------------------------------------------------------
# GPT-2
# ---------------------------------------------------------------------------

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
        n_layer = _pos_int("n_layer", _need(raw, "n_layer"))
        n_embd = _pos_int("n_embd", _need(raw, "n_embd"))
        n_head = _pos_int("n_head", _need(raw, "n_head"))
        vocab = _pos_int("vocab_size", _need(raw, "vocab_size"))
        # the reference spells the table length n_ctx (config.py:68)
        n_pos = _pos_int("n_positions", _need(raw, "n_positions", "n_ctx"))
        if "n_positions" in raw and "n_ctx" in raw and raw["n_ctx"] is not None \
                and raw["n_positions"] is not None and raw["n_ctx"] != raw["n_positions"]:
            raise ConfigError(
                f"n_positions ({raw['n_positions']}) and n_ctx ({raw['n_ctx']}) disagree")
        if n_embd % n_head:
            raise ConfigError(f"n_embd ({n_embd}) is not a multiple of n_head ({n_head})")
        n_inner = raw.get("n_inner")
        if n_inner is not None:
            n_inner = _pos_int("n_inner", n_inner)
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
            scale_attn_weights=_flag("scale_attn_weights", raw.get("scale_attn_weights", True)),
            scale_attn_by_inverse_layer_idx=_flag(
                "scale_attn_by_inverse_layer_idx",
                raw.get("scale_attn_by_inverse_layer_idx", False)),
            tie_word_embeddings=_flag("tie_word_embeddings",
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
