"""The random-weights law of the library restated with Python's own integers and floats, one
element at a time (test-side code; it shares nothing with the package's NumPy and CUDA
implementations, which must give the same bits).

key = mix(mix(seed) ^ fnv1a64(name)); pair j = element // 2: r = mix(key + (j + 1) * GAMMA);
Box-Muller with u = (2 hi + 1) / 2^33 and the angle 2 pi lo / 2^32: the logarithm through
ln f = 2 atanh((f - 1) / (f + 1)) on m = 2 hi + 1 = f 2^e, sine and cosine by octant reduction and
Taylor series, every float64 operation rounded once (Python floats never fuse a multiply with
an add). It stands where the reference draws N(0, initializer_range) from torch's generator
(src/transformers/models/falcon/modeling_falcon.py:794-808).
"""
import math
import struct

M64 = (1 << 64) - 1


def _mix(x):
    x &= M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M64
    return x ^ (x >> 31)


def _fnv(data):
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & M64
    return h


def standard_normal(seed, name, element):
    key = _mix(_mix(seed) ^ _fnv(name.encode("utf-8")))
    j = element // 2
    r = _mix(key + (j + 1) * 0x9E3779B97F4A7C15)
    hi, lo = r >> 32, r & 0xFFFFFFFF
    m = 2 * hi + 1
    e = m.bit_length() - 1
    f = float(m) / float(1 << e)
    if f > math.sqrt(2.0):
        f, e = f * 0.5, e + 1
    s = (f - 1.0) / (f + 1.0)
    s2 = s * s
    p = 1.0 / 21
    for k in range(9, -1, -1):
        p = p * s2
        p = p + 1.0 / (2 * k + 1)
    ln_f = (s * p) * 2.0
    t = float(33 - e) * math.log(2.0)
    t = t - ln_f
    radius = math.sqrt(t * 2.0)
    octant, frac = lo >> 29, lo & ((1 << 29) - 1)
    x = (frac + 0.5) * (1.0 / (1 << 29))
    if octant & 1:
        x = 1.0 - x
    a = x * (math.pi / 4.0)
    a2 = a * a
    ps = -1.0 / math.factorial(15)
    for k in range(6, -1, -1):
        ps = ps * a2
        ps = ps + (-1.0) ** k / math.factorial(2 * k + 1)
    sin_a = ps * a
    pc = 1.0 / math.factorial(16)
    for k in range(7, -1, -1):
        pc = pc * a2
        pc = pc + (-1.0) ** k / math.factorial(2 * k)
    cos_a = pc
    c, sn = (sin_a, cos_a) if octant in (1, 2, 5, 6) else (cos_a, sin_a)
    if octant in (2, 3, 4, 5):
        c = -c
    if octant >= 4:
        sn = -sn
    return radius * (c if element % 2 == 0 else sn)


def _to_f32(v):
    return struct.unpack("<f", struct.pack("<f", v))[0]


def _to_bf16(v32):
    (u,) = struct.unpack("<I", struct.pack("<f", v32))
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return struct.unpack("<f", struct.pack("<I", u))[0]


def value(seed, name, element, std=0.02, offset=0.0, bf16=False):
    """offset + std * z rounded to float32 (and on to bfloat16 with ``bf16``), as a Python float."""
    v = standard_normal(seed, name, element) * std
    v = _to_f32(v + offset)
    return _to_bf16(v) if bf16 else v
