"""Assembles a model from a :class:`ModelSpec`: builds the parts, collects the tensors
they ask for, derives what the cache must hold, and runs the schedule.

The model is the same object for every architecture; what differs is the spec.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

import torch

from .base import CacheRequest, TensorRequest, build_part
from .spec import LayerCall, LayerSpec, ModelSpec


class Block:
    """A layer: its parts and the way they are wired.

    An arrangement is a subclass that names its parts and their families in ``slots`` and
    wires them in ``forward``.  The parts are built from the layer's spec and become
    attributes of the same names.  At most one part of the mixer family may ask for a cache
    entry or a state slot (a :class:`LayerCall` addresses one of each)."""

    slots: Mapping[str, str] = {}          # part name -> family ("mixer", "feed_forward", "norm")

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        missing = [n for n in self.slots if n not in spec.parts]
        extra = [n for n in spec.parts if n not in self.slots]
        if missing or extra:
            raise ValueError(f"arrangement {spec.arrangement!r} has the parts "
                             f"{sorted(self.slots)}; missing {missing}, unknown {extra}")
        self.named = {name: build_part(family, spec.parts[name])
                      for name, family in self.slots.items()}
        for name, part in self.named.items():
            setattr(self, name, part)
        holders = [p for n, p in self.named.items() if self.slots[n] == "mixer"
                   and (p.cache_request() is not None or p.state_shape() is not None)]
        if len(holders) > 1:
            raise ValueError("a layer has two mixers that keep a cache or state; a layer call "
                             "addresses one cache entry and one state slot")
        mixers = [p for n, p in self.named.items() if self.slots[n] == "mixer"]
        self.cache_holder = holders[0] if holders else (mixers[0] if mixers else None)

    def parts(self):
        return tuple(self.named.values())

    def forward(self, ctx, x, cache) -> None:
        raise NotImplementedError


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (heteroserve/model/torch_engine.py:297-317)."""

    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, x, cache):
        h = ctx.buffer("normed", (x.shape[0], x.shape[1]), ctx.dtype)
        if self.mixer.takes_norm:           # the mixer forms norm + input projection itself
            self.mixer.forward(ctx, h, x, cache, norm=self.norm1)
        else:
            self.norm1.forward(ctx, h, x)
            self.mixer.forward(ctx, h, x, cache)
        if self.feed_forward.takes_norm:
            self.feed_forward.forward(ctx, h, x, norm=self.norm2)
        else:
            self.norm2.forward(ctx, h, x)
            self.feed_forward.forward(ctx, h, x)


_ARRANGEMENTS: dict[str, Callable[[LayerSpec], Block]] = {"pre_norm": PreNormBlock}


def register_arrangement(name: str, factory: Callable[[LayerSpec], Block], *, replace=False):
    if name in _ARRANGEMENTS and not replace:
        raise ValueError(f"arrangement {name!r} is already registered")
    _ARRANGEMENTS[name] = factory


@dataclass(frozen=True)
class CacheGroup:
    """Cache entries with the same needs share a pool of pages and a block table."""

    kv_heads: int
    head_dim: int
    window: int
    entries: tuple[int, ...]        # cache entry numbers, in pool order


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.position = build_part("position", spec.position)
        self.blocks: list[Block] = []
        for ls in spec.layers:
            if ls.arrangement not in _ARRANGEMENTS:
                raise ValueError(f"unknown arrangement {ls.arrangement!r}; "
                                 f"registered: {sorted(_ARRANGEMENTS)}")
            self.blocks.append(_ARRANGEMENTS[ls.arrangement](ls))
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.schedule: tuple[LayerCall, ...] = spec.resolved_schedule()
        self.capturable = all(part.capturable for part in self.parts())
        self._derive_cache()
        self.dtype = None
        self.device = None

    # -- structure ----------------------------------------------------------
    def parts(self):
        yield self.embedding
        yield self.position
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def tensor_requests(self) -> dict[str, TensorRequest]:
        out: dict[str, TensorRequest] = {}
        for part in self.parts():
            for name, req in part.tensor_requests().items():
                if name in out and out[name] != req:
                    raise ValueError(f"tensor {name!r} is requested twice with different "
                                     f"shapes or roles: {out[name]} and {req}")
                out[name] = req
        return out

    def _derive_cache(self) -> None:
        entry_req: dict[int, CacheRequest] = {}
        self.state_shapes: dict[int, tuple[int, ...]] = {}     # schedule index -> shape
        for idx, call in enumerate(self.schedule):
            mixer = self.blocks[call.layer].cache_holder
            if mixer is None:
                continue
            req = mixer.cache_request()
            if req is not None:
                if call.cache in entry_req and entry_req[call.cache] != req:
                    raise ValueError(f"cache entry {call.cache} is shared by mixers with "
                                     f"different needs: {entry_req[call.cache]} and {req}")
                entry_req[call.cache] = req
            shape = mixer.state_shape()
            if shape is not None:
                self.state_shapes[idx] = tuple(shape)
        groups: dict[CacheRequest, list[int]] = {}
        for entry in sorted(entry_req):
            groups.setdefault(entry_req[entry], []).append(entry)
        self.cache_groups: list[CacheGroup] = [
            CacheGroup(r.kv_heads, r.head_dim, r.window, tuple(es)) for r, es in groups.items()]
        self.entry_location: dict[int, tuple[int, int]] = {}
        for gi, g in enumerate(self.cache_groups):
            for k, e in enumerate(g.entries):
                self.entry_location[e] = (gi, k)

    def kv_bytes_per_token(self, itemsize: int) -> int:
        return sum(2 * g.kv_heads * g.head_dim * len(g.entries) * itemsize
                   for g in self.cache_groups)

    # -- weights --------------------------------------------------------------
    def bind(self, stored: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Convert the stored tensors once and hand every part its own.

        matrix/table → ``dtype`` (bfloat16 or float32); vector → float32; int → int32.
        A tensor asked for by two parts (a tied head) is converted once and shared."""
        requests = self.tensor_requests()
        converted: dict[str, torch.Tensor] = {}
        for name, req in requests.items():
            t = stored[name]
            if req.role in ("matrix", "table"):
                t = t.to(device=device, dtype=dtype)
                if req.transpose:
                    t = t.t()
            elif req.role == "vector":
                t = t.to(device=device, dtype=torch.float32)
            elif req.role == "int":
                t = t.to(device=device, dtype=torch.int32)
            else:
                raise ValueError(f"tensor {name!r}: unknown role {req.role!r}")
            converted[name] = t.contiguous()
        for part in self.parts():
            part.bind({n: converted[n] for n in part.tensor_requests()})
        self.dtype, self.device = dtype, device
        self.tensors = converted

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())

    # -- the forward pass ---------------------------------------------------
    def forward(self, ctx):
        """Run the tokens of ``ctx`` through the schedule; returns float32 logits
        ``[n_logit_rows, vocab]`` at ``ctx.logit_rows`` (None when none are wanted)."""
        spec = self.spec
        fused = getattr(ctx, "fused", None)
        if fused is not None and fused.applies(ctx):
            # single decoded tokens only, and a model the persistent kernel serves: one launch
            logits, ctx.fused_tokens = fused.run(ctx)
            return logits
        T = ctx.n_rows
        x = ctx.buffer("residual", (T, spec.width), torch.float32)
        ctx.position = self.position          # mixers ask it whether it acts on queries and keys
        self.embedding.forward(ctx, x, self.position)
        for idx, call in enumerate(self.schedule):
            ctx.call_index = idx
            cache = ctx.cache_view(call) if call.cache in self.entry_location else None
            self.blocks[call.layer].forward(ctx, x, cache)
        ctx.call_index = None
        W = ctx.n_logit_rows
        if W == 0:
            return None
        hf = ctx.buffer("final_normed", (W, spec.width), ctx.dtype)
        self.final_norm.forward(ctx, hf, x, rows=ctx.logit_rows)
        logits = ctx.buffer("logits", (W, spec.vocab_size), torch.float32)
        self.head.forward(ctx, logits, hf)
        return logits
