"""Seeded synthetic tensors in the ggml block formats of this path.

The reference measures on real model files (Llama-3.1-8B Q4_K_M, gpt-oss-20b)
that cannot be fetched here; these generators stand in for them with the same
shapes and the value distributions the benchmark definition states. Encoding is
the inverse of the reference's decoders (format/quant/dequant.go:148-174,
360-397), so every block is a valid ggml block.

numpy only: used by the tests, the smoke check and the benchmark to MAKE inputs;
nothing here evaluates a matmul.
"""
from __future__ import annotations

import numpy as np

from ._lib import BLOCK, MXFP4, Q4_0, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0


def rng_for(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _f16_bits(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).view(np.uint16)


def pack_q4k_scales(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """[..., 8] 6-bit scales and mins -> [..., 12] packed bytes (inverse of scaleMinK4)."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    for j in range(4):
        out[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        out[..., j + 4] = (m[..., j] & 63) | ((m[..., j + 4] >> 4) << 6)
        out[..., j + 8] = (sc[..., j + 4] & 0xF) | ((m[..., j + 4] & 0xF) << 4)
    return out


def q4k_from_parts(d_bits, dmin_bits, sc, m, codes) -> np.ndarray:
    """Assemble Q4_K blocks. d_bits, dmin_bits [n]; sc, m [n,8]; codes [n,256] in 0..15 -> [n,144] u8."""
    n = codes.shape[0]
    blk = np.zeros((n, 144), np.uint8)
    blk[:, 0:2] = np.asarray(d_bits, np.uint16).reshape(n, 1).view(np.uint8)
    blk[:, 2:4] = np.asarray(dmin_bits, np.uint16).reshape(n, 1).view(np.uint8)
    blk[:, 4:16] = pack_q4k_scales(sc, m)
    c = codes.astype(np.uint8).reshape(n, 4, 2, 32)  # group j, (low, high), l
    blk[:, 16:144] = (c[:, :, 0, :] | (c[:, :, 1, :] << 4)).reshape(n, 128)
    return blk


def q4k_matrix(rng: np.random.Generator, nrows: int, k: int, d_sigma: float = 0.02) -> np.ndarray:
    """Random Q4_K tensor [nrows][k/256 * 144] u8: d, dmin = f16(|N(0, d_sigma)|); sc, m ~ U{0..63};
    codes ~ U{0..15}."""
    assert k % 256 == 0
    n = nrows * (k // 256)
    d = _f16_bits(np.abs(rng.normal(0.0, d_sigma, n)).astype(np.float32))
    dmin = _f16_bits(np.abs(rng.normal(0.0, d_sigma, n)).astype(np.float32))
    sc = rng.integers(0, 64, (n, 8), dtype=np.uint8)
    m = rng.integers(0, 64, (n, 8), dtype=np.uint8)
    codes = rng.integers(0, 16, (n, 256), dtype=np.uint8)
    return q4k_from_parts(d, dmin, sc, m, codes).reshape(nrows, (k // 256) * 144)


def q8_0_from_parts(d_bits, codes) -> np.ndarray:
    n = codes.shape[0]
    blk = np.zeros((n, 34), np.uint8)
    blk[:, 0:2] = np.asarray(d_bits, np.uint16).reshape(n, 1).view(np.uint8)
    blk[:, 2:34] = codes.astype(np.int8).view(np.uint8)
    return blk


def q8_0_matrix(rng: np.random.Generator, nrows: int, k: int, d_sigma: float = 0.01) -> np.ndarray:
    """Random Q8_0 tensor [nrows][k/32 * 34] u8: codes ~ U{-127..127}, d = f16(|N(0, d_sigma)|)."""
    assert k % 32 == 0
    n = nrows * (k // 32)
    d = _f16_bits(np.abs(rng.normal(0.0, d_sigma, n)).astype(np.float32))
    codes = rng.integers(-127, 128, (n, 32), dtype=np.int8)
    return q8_0_from_parts(d, codes).reshape(nrows, (k // 32) * 34)


def mxfp4_from_parts(e, codes) -> np.ndarray:
    """e [n] u8, codes [n,32] in 0..15 -> [n,17] u8 (low nibble = element j, high = j+16)."""
    n = codes.shape[0]
    blk = np.zeros((n, 17), np.uint8)
    blk[:, 0] = e
    c = codes.astype(np.uint8)
    blk[:, 1:17] = c[:, :16] | (c[:, 16:] << 4)
    return blk


def mxfp4_matrix(rng: np.random.Generator, nrows: int, k: int, e_lo: int = -8, e_hi: int = 0) -> np.ndarray:
    """Random MXFP4 tensor [nrows][k/32 * 17] u8: e8m0 byte = 127 + U{e_lo..e_hi}, codes ~ U{0..15}."""
    assert k % 32 == 0
    n = nrows * (k // 32)
    e = (127 + rng.integers(e_lo, e_hi + 1, n)).astype(np.uint8)
    codes = rng.integers(0, 16, (n, 32), dtype=np.uint8)
    return mxfp4_from_parts(e, codes).reshape(nrows, (k // 32) * 17)


def random_blocks(rng: np.random.Generator, t: int, nrows: int, k: int, d_sigma: float = 0.02) -> np.ndarray:
    """Random tensor of a format whose every payload bit pattern is a valid code (Q4_0, Q5_0, Q5_1, Q5_K, Q6_K):
    uniform random payload bytes, and every f16 scale field = f16(|N(0, d_sigma)|) so that no value is Inf or NaN."""
    be, bb = BLOCK[t]
    nb = nrows * (k // be)
    blk = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    halves = {Q4_0: (0,), Q5_0: (0,), Q5_1: (0, 2), Q5_K: (0, 2), Q6_K: (208,)}[t]
    for off in halves:
        h = np.abs(rng.normal(0.0, d_sigma, nb)).astype(np.float16).view(np.uint16)
        blk[:, off] = h & 0xFF
        blk[:, off + 1] = h >> 8
    return blk.reshape(nrows, (k // be) * bb)


def matrix(rng: np.random.Generator, t: int, nrows: int, k: int) -> np.ndarray:
    if t in (Q4_0, Q5_0, Q5_1, Q5_K, Q6_K):
        return random_blocks(rng, t, nrows, k)
    if t == Q4_K:
        return q4k_matrix(rng, nrows, k)
    if t == Q8_0:
        return q8_0_matrix(rng, nrows, k)
    if t == MXFP4:
        return mxfp4_matrix(rng, nrows, k)
    raise ValueError(f"no generator for type {t}")


def activations(rng: np.random.Generator, ntok: int, k: int) -> np.ndarray:
    """x ~ N(0, 1), f32 [ntok][k]."""
    return rng.standard_normal((ntok, k)).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = u + 0x7FFF + ((u >> 16) & 1)
    return (r >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def planted_f16_scales() -> np.ndarray:
    """f16 bit patterns worth planting as block scales: subnormals, the smallest and largest
    normals, powers of two either side of one (cf. quant.PlantScales, format/quant/types.go:158-216)."""
    return np.array([0x0001, 0x03FF, 0x0400, 0x0401, 0x1400, 0x3800, 0x3BFF, 0x3C00, 0x3C01, 0x4000,
                     0x5640, 0x7BFF, 0x8001, 0xBC00, 0x0000, 0x2E66], np.uint16)
