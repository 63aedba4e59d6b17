"""QStream's random numbers: xorshift128+ seeded through SplitMix64
(src/sampling.c:13-38), one stream per request.

Request 0 of a call uses the seed itself, so a single request draws exactly the
reference's sequence; request i uses seed + i * 0x9E3779B97F4A7C15.  A request's draws
therefore do not depend on which other requests share its batch.
"""
from __future__ import annotations

_M = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


class XorShift128Plus:
    def __init__(self, seed: int):
        seed &= _M
        state = []
        for _ in range(2):
            seed = (seed + _GOLDEN) & _M
            seed = ((seed ^ (seed >> 30)) * 0xBF58476D1CE4E5B9) & _M
            seed = ((seed ^ (seed >> 27)) * 0x94D049BB133111EB) & _M
            s = seed ^ (seed >> 31)
            state.append(s or 1)
        self.s0, self.s1 = state

    def next_float(self) -> float:
        """Uniform in [0, 1) with 23 bits, as the reference makes it (:27-38)."""
        s0, s1 = self.s0, self.s1
        result = (s0 + s1) & _M
        s1 ^= s0
        self.s0 = (((s0 << 55) | (s0 >> 9)) ^ s1 ^ (s1 << 14)) & _M
        self.s1 = ((s1 << 36) | (s1 >> 28)) & _M
        return float(result >> 41) * (1.0 / float(1 << 23))


def request_seed(seed: int, request_index: int) -> int:
    return (int(seed) + request_index * _GOLDEN) & _M
