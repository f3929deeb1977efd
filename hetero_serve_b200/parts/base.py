"""Interfaces of the parts a model is assembled from, and their registries.

A part is built from the parameters of its :class:`PartSpec` alone.  It says which
checkpoint tensors it needs (:meth:`Part.tensor_requests`), receives them converted
and on the device (:meth:`Part.bind`) and runs on a :class:`StepContext`
(``hetero_serve_b200.engine.context``).  Five kinds exist:

========  ==================================================================
mixer     ``forward(ctx, h, x, cache)``: mixes information between the tokens
          of a request (attention here) and ADDS its result into the float32
          residual stream ``x``.  Declares what it needs cached.
feed      ``forward(ctx, h, x)``: per-token transform, added into ``x``.
norm      ``forward(ctx, out, x, rows=None)``: normalises rows of ``x``.
position  how positions enter: a table added at the embedding and/or a
          transform of queries and keys inside a mixer.
embedding / head: token table at the input, logits at the output.
========  ==================================================================

New kinds are added with the ``register_*`` functions; a test can register a toy
part and build a model around it without touching this package.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

import torch


@dataclass(frozen=True)
class TensorRequest:
    """A checkpoint tensor a part needs.

    ``role`` decides the precision it is held in: ``matrix`` and ``table`` follow the
    compute dtype (bfloat16 or float32), ``vector`` (biases, norm parameters) is always
    float32, ``int`` is int32.  ``transpose`` asks for the stored [in, out] matrix as
    [out, in], the layout the linear kernels read (done once, at binding).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    transpose: bool = False


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer wants kept per token: keys and values of ``kv_heads x head_dim``,
    all of them (``window == 0``) or the last ``window`` positions."""

    kv_heads: int
    head_dim: int
    window: int = 0


class Part:
    kind: str = ""
    # False for a part whose forward cannot be captured in a CUDA graph (its launches depend
    # on values read back to the host); a model with such a part is run without graphs.
    capturable: bool = True

    def tensor_requests(self) -> dict[str, TensorRequest]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the requested tensors, converted and on the device."""

    def fused_decode_params(self) -> dict | None:
        """What the persistent decode kernel needs of this part (its bound tensors, sizes and
        constants), or None when the part cannot run inside it.  See ``parts/fused.py``."""
        return None

    # sizes of temporary buffers are taken from the step context, nothing is allocated here


class Mixer(Part):
    # A part that sets ``takes_norm`` is handed the norm that precedes it (``norm=``) and an
    # ``h`` that is NOT yet normalised; it must form its input projection with
    # ``norm.linear(ctx, out, h, x, w, bias, act)``.  Parts that leave it False receive a
    # normalised ``h``.
    takes_norm = False

    def cache_request(self) -> CacheRequest | None:
        return None

    def state_shape(self) -> tuple[int, ...] | None:
        """Shape of the float32 state this mixer keeps per live request (fixed size), if any."""
        return None

    def forward(self, ctx, h, x, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    takes_norm = False

    def forward(self, ctx, h, x) -> None:
        raise NotImplementedError


class Norm(Part):
    def forward(self, ctx, out, x, rows=None) -> None:
        raise NotImplementedError

    def linear(self, ctx, out, h, x, w, bias=None, act="none") -> None:
        """``out = act(norm(x) @ w.T + bias)``: the input projection of the part that follows
        this norm.  The default normalises into ``h`` and projects; a norm whose kernel can be
        fused into the projection overrides it."""
        self.forward(ctx, h, x)
        ctx.ops.linear(out, h, w, bias, act=act)


class PositionEncoding(Part):
    def embedding_table(self) -> torch.Tensor | None:
        """A [max_positions, width] table added to the token embedding, or None."""
        return None

    def max_positions(self) -> int | None:
        return None

    # A position encoding that acts on queries and keys instead of (or besides) the embedding
    # sets ``acts_in_mixer`` and implements ``transform_qk``: an attention mixer calls it on its
    # projected ``qkv`` rows ([tokens, q | k | v columns], in place) before keys are appended
    # and scores are formed.  ``ctx.tok_pos`` holds the position of every row.
    acts_in_mixer = False

    def transform_qk(self, ctx, qkv, geometry) -> None:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx, x, position: PositionEncoding) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, logits, h) -> None:
        raise NotImplementedError


_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, factory: Callable[..., Part], replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    reg[kind] = factory


def register_mixer(kind, factory, *, replace=False):
    _register("mixer", kind, factory, replace)


def register_feed_forward(kind, factory, *, replace=False):
    _register("feed_forward", kind, factory, replace)


def register_norm(kind, factory, *, replace=False):
    _register("norm", kind, factory, replace)


def register_position(kind, factory, *, replace=False):
    _register("position", kind, factory, replace)


def register_embedding(kind, factory, *, replace=False):
    _register("embedding", kind, factory, replace)


def register_head(kind, factory, *, replace=False):
    _register("head", kind, factory, replace)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def build_part(family: str, spec) -> Part:
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise ValueError(f"unknown {family} kind {spec.kind!r}; registered: {sorted(reg)}")
    part = reg[spec.kind](**dict(spec.params))
    part.kind = spec.kind
    return part
