"""Seeded synthetic inputs for the parity tests and the benchmark's host-side data.

Values are approximately N(0,1) but built from integer arithmetic only (sum of twelve 16-bit
uniforms from a counter-based splitmix64 hash, centred and scaled by a power of two), so the same
(seed, stream) gives bit-identical float32 arrays on every machine and numpy build: no libm call and
no library RNG is involved.  Every value is a multiple of 2**-16 in (-6, 6).
"""
from __future__ import annotations

import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M
        return x ^ (x >> np.uint64(31))


def normal(seed: int, stream: int, shape) -> np.ndarray:
    n = int(np.prod(shape))
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        base = _mix64(np.uint64(seed) ^ _mix64(np.uint64(stream) * np.uint64(0x100000001B3) + idx))
    total = np.zeros(n, dtype=np.int64)
    h = base
    for _ in range(3):  # 3 hashes x 4 lanes of 16 bits = 12 uniforms
        for sh in (0, 16, 32, 48):
            total += ((h >> np.uint64(sh)) & np.uint64(0xFFFF)).astype(np.int64)
        h = _mix64(h)
    x = (total - 6 * 65535).astype(np.float32) / np.float32(65536.0)
    return x.reshape(shape)


def integers(seed: int, stream: int, lo: int, hi: int, shape) -> np.ndarray:
    """Uniform integers in [lo, hi] (inclusive), int32."""
    n = int(np.prod(shape))
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        h = _mix64(np.uint64(seed) ^ _mix64(np.uint64(stream) * np.uint64(0x100000001B3) + idx))
    span = np.uint64(hi - lo + 1)
    return (lo + (h % span).astype(np.int64)).astype(np.int32).reshape(shape)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16 -> float32, on the raw bits (the reference's rounding rule,
    include/uocr/common.h:56-64)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)
    return ((u & np.uint64(0xFFFF)) << np.uint64(16)).astype(np.uint32).view(np.float32).reshape(x.shape)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)
    return (u & np.uint64(0xFFFF)).astype(np.uint16).reshape(x.shape)
