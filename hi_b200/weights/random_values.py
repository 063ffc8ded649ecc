"""Seeded random numbers for weights that are the same bits wherever they are made: this
module's numpy arithmetic on the host and ``hb_random_normal`` (``hi_b200/csrc/random_fill.cu``)
on the device compute, for element ``i`` of a tensor with key ``K``,

    c = popcount of 256 hashed bits,  u = 24 more hashed bits,
    value = float32((c - 128) * 2**24 + u - 2**23) * scale

with hashed words ``mix64(K + (5 i + j + 1) * GOLDEN)``. The binomial count smoothed by the
uniform follows the normal curve with ``SIGMA_STEPS`` steps to a standard deviation; only
integer arithmetic comes before the one float multiplication, so no library function of
either side can make the two differ. (The reference has no random-weights mode.)
"""
from __future__ import annotations

import hashlib

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1
SIGMA_STEPS = float(np.sqrt(64.0 + 1.0 / 12.0))     # standard deviation of count + uniform, in steps of the count


def _mix64_int(z: int) -> int:
    z &= MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK
    z ^= z >> 31
    return z


def tensor_key(seed: int, name: str) -> int:
    """64 bits from the seed and the tensor's name."""
    digest = hashlib.sha256(name.encode()).digest()
    return _mix64_int((int(seed) & MASK) ^ int.from_bytes(digest[:8], "little"))


def scale_for(std: float) -> np.float32:
    """The float32 factor that turns the integer values into N(0, std)."""
    return np.float32(float(std) / (SIGMA_STEPS * float(1 << 24)))


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z ^ (z >> np.uint64(30))
    z = z * np.uint64(0xBF58476D1CE4E5B9)
    z = z ^ (z >> np.uint64(27))
    z = z * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def normal_values(key: int, first: int, count: int, std: float) -> np.ndarray:
    """float32 values of elements ``first .. first + count - 1``, by the host runtime (C++)."""
    from ..host import build as host

    out = np.empty(count, dtype=np.float32)
    code = host.library().hbh_random_normal(out.ctypes.data, count, first, key, float(scale_for(std)))
    if code != 0:
        raise ValueError(f"hbh_random_normal refused its arguments (code {code})")
    return out


def normal_values_numpy(key: int, first: int, count: int, std: float) -> np.ndarray:
    """The same values by numpy alone: the written-out definition that tests hold both the host
    runtime and the device kernel against."""
    out = np.empty(count, dtype=np.float32)
    scale = scale_for(std)
    golden = np.uint64(GOLDEN)
    step = 1 << 20
    with np.errstate(over="ignore"):
        for begin in range(0, count, step):
            n = min(step, count - begin)
            i = np.arange(first + begin, first + begin + n, dtype=np.uint64)
            base = np.uint64(key) + (np.uint64(5) * i + np.uint64(1)) * golden
            c = np.zeros(n, dtype=np.int64)
            for j in range(4):
                c += np.bitwise_count(_mix64(base + np.uint64(j) * golden)).astype(np.int64)
            u = (_mix64(base + np.uint64(4) * golden) >> np.uint64(40)).astype(np.int64)
            v = (c - 128) * (1 << 24) + u - (1 << 23)
            out[begin:begin + n] = v.astype(np.float32) * scale
    return out
