"""Declarative description of a model: which parts make each layer, and the
order in which layers run.

A :class:`ModelSpec` is plain data.  An architecture's builder produces it from
its typed configuration; :class:`hetero_serve_b200.parts.model.Model` turns it
into part objects through the part registries.  A part receives only the
parameters in its own :class:`PartSpec` (sizes, constants, the names of its
tensors), so no part knows which model it belongs to, and two layers of one
model may use different mixers or feed-forwards.

The order of execution is data as well: ``schedule`` is a list of
:class:`LayerCall`.  It may name a layer twice (weights shared between two
calls), and a call may read the cache another call wrote (``cache`` names the
cache entry; ``writes_cache=False`` makes the call a reader only).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


class LayerSpec:
    """One block: named parts and the arrangement that wires them.

    ``parts`` maps a name to a :class:`PartSpec`.  Which names exist, and which family
    (mixer, feed_forward, norm) each belongs to, is decided by the arrangement: the
    ``pre_norm`` arrangement built here has ``norm1``, ``mixer``, ``norm2`` and
    ``feed_forward``,

        x += mixer(norm1(x));  x += feed_forward(norm2(x))

    another arrangement may have others (one shared norm for a parallel block, norms after
    the parts, no second norm).  Parts may be given as keywords:
    ``LayerSpec(norm1=..., mixer=..., norm2=..., feed_forward=...)``.
    """

    __slots__ = ("arrangement", "parts")

    def __init__(self, arrangement: str = "pre_norm",
                 parts: Mapping[str, PartSpec] | None = None, **named: PartSpec):
        merged = dict(parts or {})
        merged.update(named)
        for name, spec in merged.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"part {name!r} of a layer must be a PartSpec, got {spec!r}")
        object.__setattr__(self, "arrangement", arrangement)
        object.__setattr__(self, "parts", MappingProxyType(merged))

    def __setattr__(self, name, value):
        raise AttributeError("a LayerSpec is immutable")

    def __getattr__(self, name):            # ls.mixer, ls.norm1, ...: the part of that name
        try:
            return object.__getattribute__(self, "parts")[name]
        except KeyError:
            raise AttributeError(f"this layer has no part named {name!r}") from None

    def __eq__(self, other):
        return (isinstance(other, LayerSpec) and self.arrangement == other.arrangement
                and dict(self.parts) == dict(other.parts))

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted((k, hash(v)) for k, v in self.parts.items()))))

    def __repr__(self):
        return f"LayerSpec({self.arrangement!r}, {dict(self.parts)!r})"


@dataclass(frozen=True)
class LayerCall:
    layer: int                    # index into ModelSpec.layers
    cache: int | None = None      # cache entry this call uses; None → one of its own
    writes_cache: bool = True     # False: only reads what an earlier call wrote


@dataclass(frozen=True)
class ModelSpec:
    name: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: int | None = None
    # how checkpoint names map onto the names the parts ask for
    strip_prefixes: tuple[str, ...] = ()
    ignore_tensors: tuple[str, ...] = ()      # regular expressions, matched after stripping

    def resolved_schedule(self) -> tuple[LayerCall, ...]:
        """The schedule with every ``cache=None`` replaced by a fresh entry index."""
        used = {c.cache for c in self.schedule if c.cache is not None}
        nxt = 0
        out = []
        for call in self.schedule:
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule names layer {call.layer}, model has {len(self.layers)}")
            if call.cache is None:
                while nxt in used:
                    nxt += 1
                used.add(nxt)
                out.append(LayerCall(call.layer, nxt, call.writes_cache))
            else:
                out.append(call)
        # entries must be numbered densely so they can index a pool
        entries = sorted({c.cache for c in out})
        if entries != list(range(len(entries))):
            raise ValueError(f"cache entries must be numbered 0..n-1 without gaps, got {entries}")
        seen_writer: set[int] = set()
        for c in out:
            if c.writes_cache:
                seen_writer.add(c.cache)
            elif c.cache not in seen_writer:
                raise ValueError(
                    f"layer call {c} reads cache entry {c.cache} before any call wrote it")
        return tuple(out)
