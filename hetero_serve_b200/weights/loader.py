"""Weights by tensor name: checking a checkpoint against what the model's parts ask
for, and the random-weights mode that writes a whole model folder.

The reference looks tensors up by name after dropping a ``transformer.``/``model.``
prefix and fails with a bare ``KeyError`` on the first missing one
(heteroserve/model/weights.py:54-100).  Here every problem of a checkpoint is
collected into one :class:`WeightError`: missing tensors, unexpected tensors and
wrong shapes.
"""

from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Mapping

import torch

from ..config.model_config import ConfigError, architecture_of, get_architecture
from .safetensors_io import SafetensorsError, read_safetensors, write_safetensors


class WeightError(ValueError):
    """A checkpoint that does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the details the message lists."""

    def __init__(self, where, missing, unexpected, wrong_shape, other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = dict(wrong_shape)
        self.other = list(other)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, (got, want) in sorted(self.wrong_shape.items()):
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def canonical_names(raw: Mapping[str, torch.Tensor], strip_prefixes, ignore_patterns):
    """Drop known prefixes and ignorable buffers; returns ``{canonical: tensor}``."""
    ignore = [re.compile(p) for p in ignore_patterns]
    out: dict[str, torch.Tensor] = {}
    clashes = []
    for name, t in raw.items():
        short = name
        for p in strip_prefixes:
            if name.startswith(p):
                short = name[len(p):]
                break
        if any(rx.fullmatch(short) for rx in ignore):
            continue
        if short in out:
            clashes.append(f"{short!r} appears twice (with and without a prefix)")
        out[short] = t
    return out, clashes


def check_tensors(where, tensors: Mapping[str, torch.Tensor], requests) -> None:
    missing = [n for n in requests if n not in tensors]
    unexpected = [n for n in tensors if n not in requests]
    wrong = {}
    other = []
    for n, req in requests.items():
        if n in tensors:
            t = tensors[n]
            if tuple(t.shape) != tuple(req.shape):
                wrong[n] = (tuple(t.shape), tuple(req.shape))
            if req.role != "int" and not t.dtype.is_floating_point:
                other.append(f"wrong type: {n} is {t.dtype}, expected a floating-point tensor")
    if missing or unexpected or wrong or other:
        raise WeightError(where, missing, unexpected, wrong, other)


def load_checkpoint(model_dir: str | Path, model) -> dict[str, torch.Tensor]:
    """Read ``model.safetensors`` of a model folder and check it against ``model``
    (a :class:`hetero_serve_b200.parts.Model`).  Tensors keep their stored type."""
    model_dir = Path(model_dir)
    path = model_dir / "model.safetensors"
    if not path.is_file():
        if (model_dir / "model.safetensors.index.json").is_file():
            raise WeightError(model_dir, [], [], {}, ["the checkpoint is sharded "
                              "(model.safetensors.index.json); only a single model.safetensors "
                              "is read"])
        raise WeightError(model_dir, [], [], {}, ["no model.safetensors in the folder"])
    try:
        raw = read_safetensors(path)
    except SafetensorsError as exc:
        raise WeightError(model_dir, [], [], {}, [str(exc)]) from None
    tensors, clashes = canonical_names(raw, model.spec.strip_prefixes, model.spec.ignore_tensors)
    if clashes:
        raise WeightError(path, [], [], {}, clashes)
    check_tensors(path, tensors, model.tensor_requests())
    return tensors


def random_weights(config: Mapping | object, seed: int) -> tuple[dict, dict[str, torch.Tensor]]:
    """``(config.json dictionary, float32 tensors)`` for a raw or typed configuration."""
    if isinstance(config, Mapping):
        arch = architecture_of(config)
        typed = arch.config_cls.from_dict(config)
    else:
        typed = config
        arch = get_architecture(typed.architectures[0])
    return typed.to_dict(), arch.init_weights(typed, seed)


def write_model_dir(out_dir: str | Path, config: Mapping | object, seed: int,
                    dtype: str | torch.dtype = "float32") -> Path:
    """The random-weights mode: write ``config.json`` and ``model.safetensors`` for a
    configuration and a seed.  ``dtype='bfloat16'`` stores matrices and tables (tensors of
    two or more dimensions) in bfloat16 and leaves vectors in float32."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cfg_dict, tensors = random_weights(config, seed)
    td = dtype if isinstance(dtype, torch.dtype) else {
        "float32": torch.float32, "fp32": torch.float32,
        "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}.get(str(dtype))
    if td is None:
        raise ConfigError(f"cannot store weights as {dtype!r}")
    if td != torch.float32:
        tensors = {n: (t.to(td) if t.dim() >= 2 else t) for n, t in tensors.items()}
    cfg_out = dict(cfg_dict)
    cfg_out["torch_dtype"] = "bfloat16" if td == torch.bfloat16 else "float32"
    (out_dir / "config.json").write_text(json.dumps(cfg_out, indent=2) + "\n")
    write_safetensors(out_dir / "model.safetensors", tensors,
                      {"format": "pt", "seed": str(seed)})
    return out_dir
