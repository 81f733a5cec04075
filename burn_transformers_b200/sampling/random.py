"""Counter-based uniforms for sampling (src/generation/random.rs:237-252 of the reference)."""
from __future__ import annotations

_MASK = (1 << 64) - 1
_GAMMA = 0x9E3779B97F4A7C15


def splitmix64(seed: int, index: int) -> int:
    """Draw `index` of the stream `seed`: mix(seed + gamma * (index + 1))."""
    v = (seed + _GAMMA * ((index + 1) & _MASK)) & _MASK
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & _MASK
    return v ^ (v >> 31)


def interior_unit_f32(bits: int) -> float:
    """The midpoint of one of 2^23 equal intervals of (0, 1): exact in float32, never 0 or 1."""
    return ((bits >> 41) + 0.5) / float(1 << 23)


def sequence_stream(seed: int, request: int) -> int:
    """Seed of the stream that request number `request` of a generate call draws from."""
    return splitmix64(seed, request)


def uniform(seed: int, index: int) -> float:
    return interior_unit_f32(splitmix64(seed, index))
