"""Named configurations for the random-weights mode.  Every registered architecture brings
its own (``Architecture.presets``); this module only looks a name up across them."""

from __future__ import annotations

from .model_config import ConfigError, _ARCHITECTURES


def _shipped() -> None:
    from .. import architectures  # noqa: F401  (registers the shipped architectures)


def _key(name: str) -> str:
    return name.lower().replace("_", "-")


def preset_names() -> list[str]:
    _shipped()
    return sorted({n for a in _ARCHITECTURES.values() for n in a.presets})


def preset(name: str) -> dict:
    """The config.json dictionary a preset name (or one of its aliases) stands for."""
    _shipped()
    key = _key(name)
    for arch in _ARCHITECTURES.values():
        k = arch.preset_aliases.get(key, key)
        if k in arch.presets:
            return dict(arch.presets[k])
    raise ConfigError(f"unknown preset {name!r}; known: {preset_names()}")
