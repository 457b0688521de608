"""The library's own generator of normal random numbers, once on the host (this file, NumPy) and
once as a CUDA kernel (csrc/fill_normal.cu). Both give the same bits for the same
(seed, tensor name, element index), so a model filled on the device equals the model folder that
the host writes from the same seed, and any slice of any tensor can be regenerated alone.

It stands where the reference draws from torch's global generator
(``_init_weights``, src/transformers/models/falcon/modeling_falcon.py:794-808).

The law. ``key = mix(mix(seed) ^ fnv1a64(name))``. Elements come in pairs: pair ``j`` holds
elements ``2j`` and ``2j + 1``. ``r = mix(key + (j + 1) * GAMMA)`` (the splitmix64 sequence);
its high 32 bits give the radius, its low 32 bits the angle of a Box-Muller transform:

* ``u = (2 hi + 1) / 2^33`` in (0, 1); ``-2 ln u`` from the integer ``m = 2 hi + 1 = f 2^e`` with
  ``f`` in (sqrt(1/2), sqrt(2)], ``ln f = 2 atanh((f - 1) / (f + 1))`` as an 11-term series;
* the angle ``2 pi lo / 2^32`` is reduced with integers to an octant (3 bits) and a place in it
  (29 bits, taken at the middle of its cell); sine and cosine of the reduced angle in
  [0, pi/4] are Taylor polynomials, mirrored and swapped by the octant.

Everything is float64 arithmetic with one rounding per operation and no fused multiply-add
(NumPy's elementwise loops here; ``__dmul_rn`` / ``__dadd_rn`` / ``__ddiv_rn`` / ``__dsqrt_rn`` in
the kernel), which IEEE 754 makes the same on every machine; no library logarithm or sine is
called. The value is ``offset + std * z``, rounded to float32 and, for bfloat16 tensors, from
there to bfloat16 (both to nearest, ties to even).
"""
from __future__ import annotations

import math
from typing import Tuple

import numpy as np

MASK64 = (1 << 64) - 1
GAMMA = 0x9E3779B97F4A7C15
MIX_A = 0xBF58476D1CE4E5B9
MIX_B = 0x94D049BB133111EB
FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3

LN2 = math.log(2.0)              # 0x1.62e42fefa39efp-1
SQRT2 = math.sqrt(2.0)           # 0x1.6a09e667f3bcdp+0
QUARTER_PI = math.pi / 4.0       # 0x1.921fb54442d18p-1
# 1/(2k+1), k = 0..10: the series of atanh
ATANH_COEF = tuple(1.0 / (2 * k + 1) for k in range(11))
# (-1)^k / (2k+1)!, k = 0..7 and (-1)^k / (2k)!, k = 0..8: Taylor series of sine and cosine
SIN_COEF = tuple((-1.0) ** k / math.factorial(2 * k + 1) for k in range(8))
COS_COEF = tuple((-1.0) ** k / math.factorial(2 * k) for k in range(9))


def fnv1a64(data: bytes) -> int:
    h = FNV_OFFSET
    for b in data:
        h = ((h ^ b) * FNV_PRIME) & MASK64
    return h


def mix_int(x: int) -> int:
    """The finaliser of splitmix64 on a Python integer."""
    x &= MASK64
    x = ((x ^ (x >> 30)) * MIX_A) & MASK64
    x = ((x ^ (x >> 27)) * MIX_B) & MASK64
    return x ^ (x >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream."""
    return mix_int(mix_int(seed) ^ fnv1a64(name.encode("utf-8")))


def _mix(x: np.ndarray) -> np.ndarray:
    x = (x ^ (x >> np.uint64(30))) * np.uint64(MIX_A)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(MIX_B)
    return x ^ (x >> np.uint64(31))


def normal_pairs(key: int, first_pair: int, n_pairs: int) -> Tuple[np.ndarray, np.ndarray]:
    """Standard normal values (z0, z1) of pairs ``first_pair .. first_pair + n_pairs - 1`` as float64."""
    j = np.arange(first_pair + 1, first_pair + 1 + n_pairs, dtype=np.uint64)
    with np.errstate(over="ignore"):
        r = _mix(np.uint64(key) + j * np.uint64(GAMMA))
    hi = (r >> np.uint64(32)).astype(np.float64)
    lo = r & np.uint64(0xFFFFFFFF)

    # radius: sqrt(-2 ln u), u = m / 2^33, m = 2 hi + 1 = f * 2^e
    m = hi * 2.0 + 1.0
    f, e = np.frexp(m)                     # m = f * 2^e, f in [0.5, 1): exact
    f = f * 2.0
    e = e - 1                              # f in [1, 2)
    big = f > SQRT2
    f = np.where(big, f * 0.5, f)
    e = np.where(big, e + 1, e)
    s = (f - 1.0) / (f + 1.0)
    s2 = s * s
    p = np.full_like(s, ATANH_COEF[10])
    for c in ATANH_COEF[9::-1]:
        p = p * s2 + c
    ln_f = (s * p) * 2.0
    t = (33 - e).astype(np.float64) * LN2 - ln_f          # -ln u
    radius = np.sqrt(t * 2.0)

    # angle: octant and place in the octant
    octant = (lo >> np.uint64(29)).astype(np.int64)
    frac = (lo & np.uint64((1 << 29) - 1)).astype(np.float64)
    x = (frac + 0.5) * (1.0 / (1 << 29))
    x = np.where(octant & 1, 1.0 - x, x)
    a = x * QUARTER_PI
    a2 = a * a
    ps = np.full_like(a, SIN_COEF[7])
    for c in SIN_COEF[6::-1]:
        ps = ps * a2 + c
    sin_a = ps * a
    pc = np.full_like(a, COS_COEF[8])
    for c in COS_COEF[7::-1]:
        pc = pc * a2 + c
    cos_a = pc
    swap = ((octant + 1) >> 1) & 1         # octants 1, 2, 5, 6: sine and cosine change places
    cos_t = np.where(swap, sin_a, cos_a)
    sin_t = np.where(swap, cos_a, sin_a)
    cos_neg = ((octant + 2) >> 2) & 1      # octants 2..5: cosine negative
    sin_neg = octant >> 2                  # octants 4..7: sine negative
    cos_t = np.where(cos_neg, -cos_t, cos_t)
    sin_t = np.where(sin_neg, -sin_t, sin_t)
    return radius * cos_t, radius * sin_t


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


def normal_values(seed: int, name: str, first: int, count: int, std: float = 0.02, offset: float = 0.0,
                  bf16: bool = False) -> np.ndarray:
    """Elements ``first .. first + count - 1`` (row-major) of the tensor ``name`` under ``seed``:
    ``offset + std * z`` as float32, rounded further to bfloat16 values with ``bf16``."""
    if count <= 0:
        return np.zeros(0, dtype=np.float32)
    key = tensor_key(seed, name)
    p0, p1 = first // 2, (first + count - 1) // 2
    out = np.empty(2 * (p1 - p0 + 1), dtype=np.float32)
    chunk = 1 << 13            # pairs per pass: the float64 temporaries stay in the cache
    for start in range(p0, p1 + 1, chunk):
        n = min(chunk, p1 + 1 - start)
        z0, z1 = normal_pairs(key, start, n)
        block = out[2 * (start - p0):2 * (start - p0 + n)]
        block[0::2] = (z0 * float(std) + float(offset)).astype(np.float32)
        block[1::2] = (z1 * float(std) + float(offset)).astype(np.float32)
    out = out[first - 2 * p0:first - 2 * p0 + count]
    return round_to_bf16(out) if bf16 else np.ascontiguousarray(out)
