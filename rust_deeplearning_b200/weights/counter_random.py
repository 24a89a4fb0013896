"""Counter-based normal random numbers: the host mirror of `csrc/random_init.cu`.

Element j of a tensor depends only on (seed, tensor name, j).  Host (numpy) and device (CUDA)
run the same sequence of IEEE-754 double operations - add, multiply, divide, square root, none of
them fused - so the float32 values agree bit for bit, and a model made on the device from
(configuration, seed) is the model a folder written on the host from the same pair holds.  The
reference's random models are unseeded (`rustml/core/main/src/core/tensor/tensor.rs:217-238`).

The recipe is in the header of `csrc/random_init.cu`: splitmix64 of key + counter gives two
uniform numbers per pair of elements, Box-Muller turns them into two normal ones; the logarithm
and the sine and cosine are short Horner sums over exactly reduced arguments.
"""
from __future__ import annotations

import numpy as np

_MASK = (1 << 64) - 1


def _mix64_int(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor: splitmix64 of the seed's hash xor the FNV-1a hash of the name."""
    h = 0xCBF29CE484222325
    for byte in name.encode():
        h = ((h ^ byte) * 0x100000001B3) & _MASK
    return _mix64_int(_mix64_int(int(seed) & _MASK) ^ h)


def _mix64(x: np.ndarray) -> np.ndarray:
    x = x + np.uint64(0x9E3779B97F4A7C15)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def _tables():
    ln_c, sin_c, cos_c = [], [], []
    f = 1.0
    for k in range(12):
        ln_c.append(1.0 / float(2 * k + 1))
        if k > 0:
            f *= float(2 * k - 1)
            f *= float(2 * k)
        sign = -1.0 if k & 1 else 1.0
        cos_c.append(sign / f)
        sin_c.append(sign / (f * float(2 * k + 1)))
    return ln_c, sin_c, cos_c


_LN_C, _SIN_C, _COS_C = _tables()
_CHUNK = 1 << 20     # pairs made at a time: bounds the temporaries


def _normal_pairs(key: int, first: int, count: int, std: float):
    """float32 (z0, z1) of pairs first .. first + count - 1."""
    with np.errstate(over="ignore"):
        i = np.arange(first, first + count, dtype=np.uint64)
        base = np.uint64(key) + np.uint64(2) * i
        a, b = _mix64(base), _mix64(base + np.uint64(1))
    u1 = ((a >> np.uint64(12)).astype(np.float64) + 0.5) * 2.220446049250313e-16
    u2 = (b >> np.uint64(11)).astype(np.float64) * 1.1102230246251565e-16
    m, e = np.frexp(u1)
    low = m < 0.7071067811865476
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e).astype(np.float64)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, _LN_C[11])
    for k in range(10, -1, -1):
        p = p * s2 + _LN_C[k]          # numpy rounds the product and the sum separately
    ln_u1 = e * 0.6931471805599453 + (2.0 * s) * p
    r = np.sqrt(-2.0 * ln_u1)
    t4 = u2 * 4.0
    q = np.floor(t4)
    t = (t4 + -q) * 1.5707963267948966
    t2 = t * t
    ps = np.full_like(t, _SIN_C[11])
    pc = np.full_like(t, _COS_C[11])
    for k in range(10, -1, -1):
        ps = ps * t2 + _SIN_C[k]
        pc = pc * t2 + _COS_C[k]
    sn, cs = t * ps, pc
    qi = q.astype(np.int64)
    c = np.choose(qi, [cs, -sn, -cs, sn])
    sv = np.choose(qi, [sn, cs, -sn, -cs])
    z0 = ((r * c) * std).astype(np.float32)
    z1 = ((r * sv) * std).astype(np.float32)
    return z0, z1


def normal(n: int, key: int, std: float) -> np.ndarray:
    """float32 [n]: N(0, std) values of the tensor with this key, element by element."""
    out = np.empty(n, dtype=np.float32)
    pairs = (n + 1) // 2
    for first in range(0, pairs, _CHUNK):
        count = min(_CHUNK, pairs - first)
        z0, z1 = _normal_pairs(key, first, count, float(std))
        lo, hi = 2 * first, min(2 * (first + count), n)
        out[lo:hi:2] = z0[: (hi - lo + 1) // 2]
        out[lo + 1:hi:2] = z1[: (hi - lo) // 2]
    return out
