"""The random-weights function, element by element, in numpy.

value(seed, tensor name, index) as the package's header states it
(mynah_slm_b200/include/mynah_random_normal.h): splitmix64's output function
of a per-tensor state and the index, two 32-bit uniforms, Box-Muller's cosine
branch with a logarithm and a cosine built from exactly rounded double
operations only. Written from that description, with numpy's element-wise
double arithmetic (which never fuses a multiply with an add); it shares no
code with the package. The reference has no random-weights mode (mynah-slm
.github/workflows/build.yml:10-13), so there is nothing of its own to cite.
"""
from __future__ import annotations

import math

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) % (1 << 64)
    return h


def mix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def log_of(u: np.ndarray) -> np.ndarray:
    bits = u.view(np.int64)
    e = ((bits >> 52) & 0x7FF) - 1022
    m = ((bits & 0x000FFFFFFFFFFFFF) | 0x3FE0000000000000).view(np.float64)
    small = m < 0.70710678118654752440
    m = np.where(small, m * 2.0, m)
    e = np.where(small, e - 1, e)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, 1.0 / 25.0)
    for d in (23, 21, 19, 17, 15, 13, 11, 9, 7, 5, 3):
        p = p * s2 + 1.0 / d
    p = p * s2 + 1.0
    return e.astype(np.float64) * 0.69314718055994530942 + (2.0 * s) * p


def sin_poly(x: np.ndarray) -> np.ndarray:
    x2 = x * x
    p = np.full_like(x, -1.0 / math.factorial(19))
    for k, sign in ((17, 1.0), (15, -1.0), (13, 1.0), (11, -1.0), (9, 1.0), (7, -1.0), (5, 1.0), (3, -1.0)):
        p = p * x2 + sign / float(math.factorial(k))
    p = p * x2 + 1.0
    return x * p


def cos_poly(x: np.ndarray) -> np.ndarray:
    x2 = x * x
    p = np.full_like(x, -1.0 / math.factorial(18))
    for k, sign in ((16, 1.0), (14, -1.0), (12, 1.0), (10, -1.0), (8, 1.0), (6, -1.0), (4, 1.0), (2, -1.0)):
        p = p * x2 + sign / float(math.factorial(k))
    return p * x2 + 1.0


def cos_turn(k: np.ndarray) -> np.ndarray:
    """cos(2 pi k / 2^32) for uint64 k < 2^32."""
    quadrant = (k >> np.uint64(30)).astype(np.int64)
    g = (k & np.uint64(0x3FFFFFFF)).astype(np.float64) * (1.0 / 1073741824.0)
    fold = g > 0.5
    a = np.where(fold, 1.0 + -g, g) * 1.57079632679489661923
    sa, ca = sin_poly(a), cos_poly(a)
    c = np.where(fold, sa, ca)
    s = np.where(fold, ca, sa)
    return np.select([quadrant == 0, quadrant == 1, quadrant == 2], [c, -s, -c], s)


def normal(seed: int, name: str, index: np.ndarray) -> np.ndarray:
    """Standard normal numbers (float64) of the elements `index` of tensor `name`."""
    index = np.asarray(index, dtype=np.uint64)
    with np.errstate(over="ignore"):
        state = mix64(np.asarray([np.uint64(seed % (1 << 64)) + GAMMA], dtype=np.uint64))[0] ^ np.uint64(fnv1a64(name))
        z = mix64(state + (index + np.uint64(1)) * GAMMA)
    u1 = ((z >> np.uint64(32)).astype(np.float64) + 1.0) * (1.0 / 4294967296.0)
    r = np.sqrt(-2.0 * log_of(u1))
    return r * cos_turn(z & np.uint64(0xFFFFFFFF))


def values(seed: int, name: str, index, mean: float, std: float, bf16: bool) -> np.ndarray:
    """float32 values as stored; with `bf16` rounded to bfloat16 (nearest, ties to even) and widened again."""
    v = (mean + std * normal(seed, name, index)).astype(np.float32)
    if bf16:
        u = v.view(np.uint32)
        u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
        v = u.view(np.float32)
    return v
