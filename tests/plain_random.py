"""The random-weights generator, written out one element at a time in plain Python.

This is the tests' statement of what ``trapetum_b200.weights.random_init`` (numpy, for model
folders) and ``csrc/random_init.cu`` (on the device) must produce, bit for bit.  It shares no code
with either.  The reference builds its synthetic models from a seeded xorshift generator inside the
program (runtime/src/lib.rs:1604-1629, runtime/src/bin/model.rs:158-177); here the generator is
counter-based, so that element ``i`` of tensor ``name`` can be made anywhere, in any order:

* key: 64-bit FNV-1a hash of the tensor's name, xor-ed with the seed, as two 32-bit words;
* Philox-4x32 with 10 rounds on the counter (i // 4, 0x54524150, 0) gives four 32-bit words;
* words (0, 1) and (2, 3) each make two normal numbers by Box and Muller's transform:
  radius from the upper 24 bits of the first word, angle from the upper 26 bits of the second;
* the logarithm, sine and cosine are short polynomials evaluated with single-precision
  additions, multiplications and divisions only, each rounded to nearest (no fused multiply-add),
  so that every machine gets the same bits;
* value = normal * std in single precision, rounded to bfloat16 (nearest, ties to even).
"""
import numpy as np

F = np.float32
MASK = 0xFFFFFFFF
M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def key_of(seed: int, name: str):
    h = fnv1a64(name) ^ (int(seed) & 0xFFFFFFFFFFFFFFFF)
    return h & MASK, (h >> 32) & MASK


def philox(c0, c1, c2, c3, k0, k1):
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & MASK, p1 & MASK, ((p0 >> 32) ^ c3 ^ k1) & MASK, p0 & MASK
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c0, c1, c2, c3


def neg_log_unit(w: int) -> np.float32:
    """-ln(u) for u = ((w >> 8) + 1) / 2^24 in (0, 1]."""
    k = (w >> 8) + 1
    e = k.bit_length() - 1
    m = F(k) / F(1 << e)                               # in [1, 2), exact
    s = (m - F(1.0)) / (m + F(1.0))
    z = s * s
    p = F(0.0909090936)
    for c in (0.111111112, 0.142857149, 0.200000003, 0.333333343):
        p = p * z + F(c)
    p = p * z + F(1.0)
    ln_m = F(2.0) * (s * p)
    return F(24 - e) * F(0.693147182) - ln_m


def sin_cos_turn(w: int):
    """(sin, cos) of 2*pi*(w >> 6) / 2^26: the top two bits pick the quadrant, the next 24 the angle in it."""
    q = w >> 30
    t = F((w >> 6) & 0xFFFFFF) * F(2.0 ** -24) * F(1.57079637)
    z = t * t
    s = F(1.60590444e-10)
    for c in (-2.50521079e-08, 2.75573188e-06, -0.000198412701, 0.00833333377, -0.166666672):
        s = s * z + F(c)
    s = (s * z + F(1.0)) * t
    c_ = F(2.08767559e-09)
    for c in (-2.755732e-07, 2.48015876e-05, -0.00138888892, 0.0416666679, -0.5):
        c_ = c_ * z + F(c)
    c_ = c_ * z + F(1.0)
    return [(s, c_), (c_, -s), (-s, -c_), (-c_, s)][q]


def to_bf16_bits(x: np.float32) -> int:
    u = int(np.asarray(x, dtype=np.float32).view(np.uint32))
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def element(seed: int, name: str, i: int, std: float) -> np.float32:
    """Element ``i`` (row-major) of tensor ``name``: a float32 that holds a bfloat16 value."""
    k0, k1 = key_of(seed, name)
    blk = i // 4
    w = philox(blk & MASK, (blk >> 32) & MASK, 0x54524150, 0, k0, k1)
    a, b = (w[0], w[1]) if (i % 4) < 2 else (w[2], w[3])
    r = np.sqrt(F(2.0) * neg_log_unit(a))
    s, c = sin_cos_turn(b)
    n = r * (c if i % 2 == 0 else s)
    v = n * F(std)
    return np.asarray(to_bf16_bits(v) << 16, dtype=np.uint32).view(np.float32)[()]
