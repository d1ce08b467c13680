"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset or model bundle is involved).

Generator: counter-based splitmix64.  Element i of stream `seed` is
mix(seed + (i + 1) * 0x9E3779B97F4A7C15) with the standard splitmix64 finaliser;
uniforms take the top 53 bits; normals are Box-Muller over two streams.
Everything is vectorised numpy and reproducible across machines.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """n outputs of the stream `seed`, starting at element `offset`."""
    with np.errstate(over="ignore"):
        i = np.arange(offset + 1, offset + n + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    u = (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))
    return lo + (hi - lo) * u


def normal(seed: int, n: int) -> np.ndarray:
    m = (n + 1) // 2
    u1 = 1.0 - uniform(seed, m)            # (0, 1]
    u2 = uniform(seed ^ 0x5DEECE66D, m)
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * m, dtype=np.float64)
    out[0::2] = r * np.cos(2 * np.pi * u2)
    out[1::2] = r * np.sin(2 * np.pi * u2)
    return out[:n]


def normal_f16(shape, seed: int, scale: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    return (normal(seed, n) * scale).astype(np.float16).reshape(shape)


def q4_0_weights(rows: int, cols: int, seed: int, d_lo: float = 0.001, d_hi: float = 0.02) -> np.ndarray:
    """GGUF Q4_0 blocks, row-major [rows, cols/32] x 18 bytes: f16 d ~ U[d_lo, d_hi],
    16 code bytes uniform 0..255 (nibbles uniform 0..15). Returns uint8 [rows * cols/32 * 18]."""
    assert cols % 32 == 0
    nblk = rows * (cols // 32)
    out = np.empty((nblk, 18), dtype=np.uint8)
    d = uniform(seed, nblk, d_lo, d_hi).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    out[:, 2:18] = splitmix64(seed ^ 0xA5A5A5A5, nblk * 2).view(np.uint8).reshape(nblk, 16)
    return out.reshape(-1)


def tq2_0_weights(rows: int, cols: int, seed: int, d_lo: float = 0.005, d_hi: float = 0.05,
                  ncodes: int = 3) -> np.ndarray:
    """GGUF TQ2_0 blocks, row-major [rows, cols/256] x 66 bytes: 64 qs bytes then f16 d.
    Codes are uniform over {0..ncodes-1} (3 = ternary, 4 also exercises the legal code 3).
    Element (j>>5)*128 + l*32 + (j&31) of a block sits in bits 2l..2l+1 of qs[j]."""
    assert cols % 256 == 0
    nblk = rows * (cols // 256)
    r = splitmix64(seed ^ 0x7E57, nblk * 64).view(np.uint16).reshape(nblk, 256)
    codes = (r % np.uint16(ncodes)).astype(np.uint8).reshape(nblk, 2, 4, 32)  # [j>>5, l, j&31]
    qs = (codes[:, :, 0, :] | (codes[:, :, 1, :] << 2) | (codes[:, :, 2, :] << 4) | (codes[:, :, 3, :] << 6))
    out = np.empty((nblk, 66), dtype=np.uint8)
    out[:, 0:64] = qs.reshape(nblk, 64)
    d = uniform(seed, nblk, d_lo, d_hi).astype(np.float16)
    out[:, 64:66] = d.view(np.uint8).reshape(nblk, 2)
    return out.reshape(-1)


def lognormal_contexts(n: int, seed: int, median: float = 2048.0, sigma: float = 1.0, lo: int = 16,
                       hi: int = 131072) -> np.ndarray:
    """Context lengths round(exp(N(ln median, sigma))) clipped to [lo, hi]."""
    x = np.exp(np.log(median) + sigma * normal(seed, n))
    return np.clip(np.rint(x), lo, hi).astype(np.uint32)
