"""The sampling rule of the engine, stated on the host.

For a request with ``seed``, the token that will take position ``p`` of the sequence is
drawn with ONE uniform number ``u = uniform_for_position(seed, p)``: the first output
word of Philox-4x32-10 with key ``(seed & 0xffffffff, seed >> 32)`` and counter
``(p, 0, 0, 0)``, its top 24 bits scaled to [0, 1).  With temperature ``T > 0`` the token
is the first index ``i`` with ``sum_{j<=i} w_j > u * sum_j w_j`` where
``w_j = exp(logit_j / T - max)`` over all tokens, or over the ``top_k`` largest logits
(ties at the threshold to the lower index) when ``0 < top_k < vocab``; with ``T <= 0``
it is the argmax (lowest index on ties).  The reference draws with numpy's generator
reseeded per token (heteroserve/worker/worker.py:43-50, 647, 694); keying the draw on
(seed, position) keeps its property that batching and preemption do not change what
is sampled.
"""

from __future__ import annotations

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32_10(counter, key):
    c = [int(x) & _MASK for x in counter]
    k = [int(x) & _MASK for x in key]
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _MASK, p1 & _MASK,
             ((p0 >> 32) ^ c[3] ^ k[1]) & _MASK, p0 & _MASK]
        k = [(k[0] + _W0) & _MASK, (k[1] + _W1) & _MASK]
    return c


def uniform_for_position(seed: int, position: int) -> float:
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    word = philox4x32_10([position, 0, 0, 0], [seed & _MASK, seed >> 32])[0]
    return (word >> 8) / 16777216.0
