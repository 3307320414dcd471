"""Seeded synthetic inputs (numpy, host side).

Values are drawn from counter-based Philox streams keyed by (seed, tensor id,
row chunk), so any row range of a tensor can be regenerated independently: a
GPU that owns rows [r0, r1) of A produces exactly the values the CPU oracle
sees for those rows.  Chunks are CHUNK_ROWS rows; shard boundaries must fall on
chunk boundaries.

Encodings: fp16 by numpy (round to nearest even); bf16 and e4m3 by the bit
routines below (round to nearest even, e4m3 saturating at +-448); xf32 by
clearing the low 13 mantissa bits (the reference's truncating conversion,
rocWMMA internal/rocwmma_xfloat32.hpp:198-203).
"""
from __future__ import annotations

import numpy as np

F16, BF16, E4M3, I8, F32, XF32, F64, I32, E5M2 = range(9)
CHUNK_ROWS = 128

NP_DTYPE = {F16: np.float16, BF16: np.uint16, E4M3: np.uint8, I8: np.int8, F32: np.float32,
            XF32: np.float32, F64: np.float64, I32: np.int32, E5M2: np.uint8}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    out = np.where(nan, (u >> 16) | 0x40, rounded)
    return out.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> OCP e4m3 bits, round to nearest even, saturate to +-448."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = ((x.view(np.uint32) >> 24) & 0x80).astype(np.uint8)
    a = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0))).astype(np.int64)
    e = np.maximum(e, -6)
    q = np.rint(a * np.exp2(3 - e)).astype(np.int64)  # np.rint rounds half to even
    carry = q == 16
    q = np.where(carry, 8, q)
    e = np.where(carry, e + 1, e)
    normal = q >= 8
    bits = np.where(normal, ((e + 7) << 3) | (q - 8), q)
    out = bits.astype(np.uint8)
    out = np.where(a >= 448.0, 0x7E, out).astype(np.uint8)
    out = np.where(a < 2.0 ** -10, 0, out).astype(np.uint8)
    out = np.where(np.isnan(x), 0x7F, out).astype(np.uint8)
    return out | sign


def e4m3_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = b.astype(np.uint32)
    s, e, m = b >> 7, (b >> 3) & 0xF, b & 7
    val = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7))
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return np.where(s == 1, -val, val).astype(np.float32)


def f32_to_e5m2_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> OCP e5m2 bits, round to nearest even, saturate to +-57344 (no infinities)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = ((x.view(np.uint32) >> 24) & 0x80).astype(np.uint8)
    a = np.abs(x).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0))).astype(np.int64)
    e = np.maximum(e, -14)
    q = np.rint(a * np.exp2(2 - e)).astype(np.int64)
    carry = q == 8
    q = np.where(carry, 4, q)
    e = np.where(carry, e + 1, e)
    bits = np.where(q >= 4, ((e + 15) << 2) | (q - 4), q)
    out = bits.astype(np.uint8)
    out = np.where(a >= 57344.0, 0x7B, out).astype(np.uint8)
    out = np.where(a < 2.0 ** -17, 0, out).astype(np.uint8)
    out = np.where(np.isnan(x), 0x7F, out).astype(np.uint8)
    return out | sign


def e5m2_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """e5m2 is the upper byte of a binary16 number."""
    return (b.astype(np.uint16) << 8).view(np.float16).astype(np.float32)


def truncate_xf32(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


def _rng(seed: int, tensor_id: int, chunk: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[(seed << 16) ^ tensor_id, chunk]))


def _encode(x: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F16:
        return x.astype(np.float16)
    if dtype == BF16:
        return f32_to_bf16_bits(x.astype(np.float32))
    if dtype == E4M3:
        return f32_to_e4m3_bits(x.astype(np.float32))
    if dtype == E5M2:
        return f32_to_e5m2_bits(x.astype(np.float32))
    if dtype == XF32:
        return truncate_xf32(x.astype(np.float32))
    if dtype == F32:
        return x.astype(np.float32)
    if dtype == F64:
        return x.astype(np.float64)
    raise ValueError(dtype)


def _fill_chunk(out, r, n, seed, tensor_id, dtype, row0, ncols, dist, scale):
    g = _rng(seed, tensor_id, (row0 + r) // CHUNK_ROWS)
    if dist == "uniform":
        out[r:r + n] = _encode(g.uniform(-1.0, 1.0, (n, ncols)), dtype)
    elif dist == "normal":
        out[r:r + n] = _encode(g.standard_normal((n, ncols)) * scale, dtype)
    elif dist == "int8":
        out[r:r + n] = g.integers(-128, 128, (n, ncols), dtype=np.int8)
    elif dist == "int32":
        out[r:r + n] = g.integers(-100, 101, (n, ncols)).astype(np.int32)
    elif dist == "pattern":
        idx = (np.arange(row0 + r, row0 + r + n)[:, None] * ncols + np.arange(ncols)[None, :])
        v = (idx % 5).astype(np.float64)
        v = np.where(idx % 3 != 0, -v, v)
        out[r:r + n] = v.astype(NP_DTYPE[dtype]) if dtype in (I8, I32) else _encode(v, dtype)
    else:
        raise ValueError(dist)


def rows(seed: int, tensor_id: int, dtype: int, row0: int, nrows: int, ncols: int,
         dist: str = "uniform", scale: float = 1.0, threads: int = 1) -> np.ndarray:
    """Rows [row0, row0+nrows) of a (?, ncols) tensor stored row by row.

    dist: "uniform" in [-1, 1]; "normal" N(0,1) * scale; "int8" uniform integers in
    [-128, 127]; "int32" small integers in [-100, 100]; "pattern" = the reference's
    small-integer fill (rocWMMA test/common.hpp:248-270: (index % 5), negated when
    index % 3 != 0), which makes every GEMM exactly representable.
    threads > 1 fills the 128-row chunks from a thread pool (every chunk has its own
    stream, so the values do not depend on the thread count).
    """
    assert row0 % CHUNK_ROWS == 0, "shards start on chunk boundaries"
    out = np.empty((nrows, ncols), dtype=NP_DTYPE[dtype])
    starts = range(0, nrows, CHUNK_ROWS)
    args = (seed, tensor_id, dtype, row0, ncols, dist, scale)
    if threads > 1 and len(starts) > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=threads) as ex:
            list(ex.map(lambda r: _fill_chunk(out, r, min(CHUNK_ROWS, nrows - r), *args), starts))
    else:
        for r in starts:
            _fill_chunk(out, r, min(CHUNK_ROWS, nrows - r), *args)
    return out


def matrix(seed: int, tensor_id: int, dtype: int, nrows: int, ncols: int, **kw) -> np.ndarray:
    """Whole (nrows, ncols) tensor, flat."""
    return rows(seed, tensor_id, dtype, 0, nrows, ncols, **kw).reshape(-1)
