"""hetero_serve_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and architecture registry, weights by tensor name, a model assembled
from parts, a paged cache with prefix reuse, one step function over ragged batches,
a continuous-batching scheduler, device-side sampling, and hand-written CUDA kernels.
"""

from . import architectures  # noqa: F401
from .config import EngineConfig, preset
from .engine import LLMEngine, Request, RequestRecord, Runner, StepEntry

__version__ = "0.1.0"
__all__ = ["EngineConfig", "LLMEngine", "Request", "RequestRecord", "Runner",
           "StepEntry", "preset"]
