"""Seeded synthetic tensors that a C++ program can reproduce bit for bit.

numpy's generators cannot be re-created from C++ and normal deviates through log/cos differ in the last place
between math libraries, so the model configurations draw their weights from a counter-based generator built from
integer arithmetic and IEEE additions only:

  u_k     = splitmix64(seed, k)  >> 11  times 2^-53          uniform on [0, 1), k = 1, 2, ...
  normal  = (u_1 + u_2 + ... + u_12) - 6                       Irwin-Hall: mean 0, variance 1, |x| <= 6

(added left to right in double precision).  oracle/ref_emit.cxx holds the same three lines in C++ and builds the
reference's own models from them, so both sides of a parity test see identical weights without shipping them.
Each tensor takes a seed of its own: tensor_seed(base, index).
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def tensor_seed(base: int, index: int) -> int:
    return (base * 1000003 + index * 7919 + 12345) & 0xFFFFFFFFFFFFFFFF


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int) -> np.ndarray:
    """n doubles on [0, 1): draws 1 .. n of the stream `seed`."""
    with np.errstate(over="ignore"):
        k = np.arange(1, n + 1, dtype=np.uint64)
        z = _mix(np.uint64(seed) + k * _GAMMA)
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed: int, n: int) -> np.ndarray:
    """n doubles, each the sum of 12 consecutive uniforms minus 6 (draws 12 i + 1 .. 12 i + 12 for value i)."""
    u = uniform(seed, 12 * n).reshape(n, 12)
    a = u[:, 0].copy()
    for j in range(1, 12):
        a = a + u[:, j]
    return a - 6.0


def normal_f32(seed: int, shape, std: float) -> np.ndarray:
    """float(std * normal) in the given shape; `std` is a double."""
    n = int(np.prod(shape))
    return (normal(seed, n) * float(std)).astype(np.float32).reshape(shape)


def uniform_f32(seed: int, shape, lo: float, hi: float) -> np.ndarray:
    """float(lo + (hi - lo) * uniform) in the given shape."""
    n = int(np.prod(shape))
    return (float(lo) + (float(hi) - float(lo)) * uniform(seed, n)).astype(np.float32).reshape(shape)
