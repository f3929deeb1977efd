"""Sampling.  Token selection runs on the device inside the step (``ops.sample``:
argmax, temperature, top-k; ``csrc/sampling.cu``).  This module holds the host-side
statement of the same rule, used to document and cross-check it.
"""

from .rule import philox4x32_10, uniform_for_position

__all__ = ["philox4x32_10", "uniform_for_position"]
