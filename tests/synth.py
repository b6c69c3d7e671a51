"""Seeded synthetic inputs shared by the parity tests and the fixture generator.

Counter-based (splitmix64 of seed and element index) so any slice of a stream can
be produced independently and the same values come out on every machine with the
same numpy build; normals come from Box-Muller in float64, rounded to float32.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix(z):
    z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def bits(seed, stream, n, start=0):
    """n 64-bit words of stream `stream` under `seed`, beginning at element `start`."""
    with np.errstate(over="ignore"):
        base = _splitmix(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream))
        idx = np.arange(start, start + n, dtype=np.uint64)
        return _splitmix(base ^ (idx * np.uint64(0xD6E8FEB86659FD93) & _M64))


def uniform(seed, stream, n, start=0):
    """float64 in (0,1)."""
    return ((bits(seed, stream, n, start) >> np.uint64(11)).astype(np.float64) + 0.5) / 9007199254740992.0


def normal(seed, stream, shape, std=1.0):
    """float32 N(0, std^2) of the given shape."""
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    step = 1 << 22
    for s in range(0, n, step):
        m = min(step, n - s)
        u1 = uniform(seed, 2 * stream, m, s)
        u2 = uniform(seed, 2 * stream + 1, m, s)
        out[s:s + m] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)
    return out.reshape(shape)


def token_ids(seed, stream, n, vocab):
    return (bits(seed, stream, n) % np.uint64(vocab)).astype(np.int64)


def lcg_uniform(seed, n):
    """The LCG the reference's own tests use (test/test_array.cpp:768-773, 817-821):
    st = st*1664525 + 1013904223;  x = (int)(st>>9) / 2^22 - 1."""
    out = np.empty(n, np.float32)
    st = seed & 0xFFFFFFFF
    for i in range(n):
        st = (st * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(st >> 9) / np.float32(1 << 22) - np.float32(1.0))
    return out
