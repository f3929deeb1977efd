"""The architecture registry, and helpers for typed model configurations.

A model folder carries a ``config.json`` in the architecture's own vocabulary.  Each
architecture lives in a module of its own under ``hetero_serve_b200/architectures/`` (or
anywhere else) and registers

* a frozen dataclass that reads and validates its keys,
* a builder that turns the typed configuration into a :class:`ModelSpec`
  (``hetero_serve_b200.parts.spec``): a purely declarative description of the
  layers, their parts and the order in which they run,
* a seeded random initialisation, and
* named configurations (presets) for the random-weights mode.

This module knows no architecture by name.

Nothing else in the framework looks at ``config.json``; every size and
constant reaches the kernels through the spec.

The typed-dataclass manner follows the reference's ``ModelConfig``
(heteroserve/config.py:21-70), which reads ``n_layer``, ``n_head``, ``n_embd``,
``vocab_size``, ``n_ctx`` and ``layer_norm_epsilon``; the reference has no
registry (it picks the model with a string compare, heteroserve/worker/worker.py:832).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
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
    # named config.json dictionaries for the random-weights mode, and other spellings of
    # their names ({alias: preset name})
    presets: Mapping[str, Mapping[str, Any]] = field(default_factory=dict)
    preset_aliases: Mapping[str, str] = field(default_factory=dict)


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


def need(raw: Mapping[str, Any], key: str, *alts: str):
    for k in (key, *alts):
        if k in raw and raw[k] is not None:
            return raw[k]
    names = " or ".join(repr(k) for k in (key, *alts))
    raise ConfigError(f"config.json is missing {names}")


def positive_int(name: str, v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {v!r}")
    return v


def flag(name: str, v: Any) -> bool:
    if not isinstance(v, bool):
        raise ConfigError(f"{name} must be true or false, got {v!r}")
    return v
