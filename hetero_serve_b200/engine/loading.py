"""From a model folder to a bound model: config.json picks the architecture, the
architecture builds the spec, the parts say which tensors they need, the loader
checks the checkpoint against that, and the model converts and keeps them."""

from __future__ import annotations

from pathlib import Path

import torch

from .. import architectures  # noqa: F401  (registers the shipped architectures)
from ..config import canonical_dtype, load_model_config
from ..parts import Model
from ..weights import load_checkpoint

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def load_model(model_dir: str | Path, dtype: str, device) -> tuple[Model, object]:
    """Returns ``(model, typed config)`` with the weights on ``device`` in ``dtype``."""
    arch, cfg = load_model_config(model_dir)
    model = Model(arch.build_spec(cfg))
    stored = load_checkpoint(model_dir, model)
    model.bind(stored, TORCH_DTYPES[canonical_dtype(dtype)], torch.device(device))
    return model, cfg
