"""The random-weights rule written out in numpy, for the tests: value = f(key, element index).

It restates the arithmetic that the package's host and device code must both follow (64 bits per
element from the splitmix64 finalizer; Box-Muller with ln and cos from their series in IEEE double
operations rounded one by one; norm gains uniform), shares no code with either, and is compared with
them bit for bit.  The distributions are those of the reference's weight script (matrices and the
embedding N(0, 0.02): scripts/synthetic_checkpoint.py:135-152), norm gains 1 + U(-0.1, 0.1).
"""
import hashlib
from math import factorial

import numpy as np

U64 = np.uint64
MASK = (1 << 64) - 1


def _mix64_int(z):
    z &= MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def tensor_key(seed, name):
    h = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")
    return _mix64_int((seed & MASK) ^ _mix64_int(h))


def element_bits(key, index):
    with np.errstate(over="ignore"):
        z = U64(key) + (np.asarray(index, dtype=U64) + U64(1)) * U64(0x9E3779B97F4A7C15)
        z = z ^ (z >> U64(30))
        z = z * U64(0xBF58476D1CE4E5B9)
        z = z ^ (z >> U64(27))
        z = z * U64(0x94D049BB133111EB)
        return z ^ (z >> U64(31))


def _ln(x):
    b = x.view(U64)
    e = ((b >> U64(52)) & U64(0x7ff)).astype(np.int64) - 1022
    m = ((b & U64(0x000fffffffffffff)) | U64(0x3fe0000000000000)).view(np.float64)
    low = m < 0.70710678118654752
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e)
    z = (m + -1.0) / (m + 1.0)
    z2 = z * z
    s = np.full_like(z, 2.0 / 21.0)
    for k in (19, 17, 15, 13, 11, 9, 7, 5, 3):
        s = s * z2 + 2.0 / k
    s = s * z2 + 2.0
    return e.astype(np.float64) * 0.69314718055994531 + s * z


def _cos_turn(k):
    k = k.astype(np.uint32)
    quadrant = k >> np.uint32(30)
    f = k & np.uint32(0x3fffffff)
    mirror = f > np.uint32(0x20000000)
    f = np.where(mirror, np.uint32(0x40000000) - f, f)
    x = f.astype(np.float64) * (1.5707963267948966 / 1073741824.0)
    x2 = x * x
    c = np.full_like(x, 1.0 / factorial(16))
    for n, sign in ((14, -1), (12, 1), (10, -1), (8, 1), (6, -1), (4, 1)):
        c = c * x2 + sign * 1.0 / factorial(n)
    c = c * x2 + -0.5
    c = c * x2 + 1.0
    s = np.full_like(x, 1.0 / factorial(17))
    for n, sign in ((15, -1), (13, 1), (11, -1), (9, 1), (7, -1), (5, 1), (3, -1)):
        s = s * x2 + sign * 1.0 / factorial(n)
    s = s * x2 + 1.0
    s = s * x
    cos_a, sin_a = np.where(mirror, s, c), np.where(mirror, c, s)
    return np.select([quadrant == 0, quadrant == 1, quadrant == 2], [cos_a, -sin_a, -cos_a], sin_a)


def normal(key, index, std=0.02):
    h = element_bits(key, index)
    u1 = ((h >> U64(32)).astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
    r = np.sqrt(-2.0 * _ln(u1))
    return ((r * _cos_turn(h & U64(0xffffffff))) * std).astype(np.float32)


def uniform(key, index, mid=1.0, width=0.2):
    h = element_bits(key, index)
    u = (h >> U64(40)).astype(np.float64) * (1.0 / 16777216.0)
    return (mid + (u * width + width * -0.5)).astype(np.float32)
