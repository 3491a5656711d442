"""The per-request random draws: one uniform number in [0, 1) per sampled token.

The draw for the k-th sampled token of a request is a pure function of the
request's seed and k (a counter-based generator: two rounds of the splitmix64
finaliser), so a request that is evicted and recomputed continues with the same
draws, and the CPU and the GPU see the same number.  The reference draws one
f32 per token from a per-request generator
(crates/llm-native-runtime/src/native_text/generation.rs:291-332).
"""
from __future__ import annotations

import os

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def draw(seed: int, counter: int) -> float:
    """Uniform in [0, 1) with 24 random bits (exactly representable in 32-bit floats)."""
    bits = _mix(_mix(seed & _MASK) ^ (counter & _MASK))
    return (bits >> 40) / float(1 << 24)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")
