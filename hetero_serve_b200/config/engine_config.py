"""Engine-side configuration: cache geometry, batching limits, precision.

Names and defaults follow the reference where it has them:
``KVConfig(block_size=16, num_blocks=512)`` (heteroserve/config.py:101-119) and
``WorkerConfig(max_batch=8, max_prefill_tokens=512)`` (heteroserve/config.py:156-165;
the worker's command line defaults the latter to 256, heteroserve/worker/worker.py:858,
and ``--max-ctx`` to 512, worker.py:859).
"""

from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError

DTYPES = ("bfloat16", "float32")
POLICIES = ("prefill_first", "mixed")


def canonical_dtype(name: str) -> str:
    alias = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32",
             "float32": "float32", "f32": "float32"}
    try:
        return alias[str(name).lower()]
    except KeyError:
        raise ConfigError(f"dtype must be one of {DTYPES}, got {name!r}") from None


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"           # "bfloat16": serving kernels; "float32": true 32-bit
    block_size: int = 16              # tokens per cache page
    num_blocks: int = 512             # pages in the pool
    max_batch: int = 8                # most requests decoded in one step
    max_prefill_tokens: int = 256     # most prompt tokens one step takes (the token budget)
    max_ctx: int | None = None        # cap on prompt + generated tokens (None: the model's)
    max_requests: int | None = None   # live requests (state slots); None → max(max_batch, 4)
    policy: str = "prefill_first"     # "prefill_first" as the reference, or "mixed"
    prefix_cache: bool = True         # reuse pages of equal prompt prefixes
    cuda_graphs: bool = True          # replay captured steps for repeated shapes
    pipeline: bool = True             # launch a step before the previous step's tokens are read
    fused_decode: bool = False        # pure decode steps of up to 16 tokens as one persistent kernel
    seed: int = 0
    device: str = "cuda:0"

    def __post_init__(self):
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype))
        if self.block_size <= 0 or self.block_size % 16:
            raise ConfigError(f"block_size must be a positive multiple of 16, got {self.block_size}")
        for name in ("num_blocks", "max_batch", "max_prefill_tokens"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.policy not in POLICIES:
            raise ConfigError(f"policy must be one of {POLICIES}, got {self.policy!r}")

    @property
    def live_requests(self) -> int:
        return self.max_requests if self.max_requests is not None else max(self.max_batch, 4)

    @property
    def capacity_tokens(self) -> int:
        return self.block_size * self.num_blocks
