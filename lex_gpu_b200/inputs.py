"""Seeded synthetic inputs for `gemm_fp4`, in the shapes and value distributions of the
benchmark configurations.  Real checkpoints are not needed for this operator.

Layout of one weight matrix (crates/lex-front/lx/gemm_fp4.lx:16-22):
  wq u8[n, k/2]   two E2M1 codes per byte, even column in the low nibble
  ws u8[n, k/16]  one E4M3 (OCP e4m3fn) scale per 16 weights
  wg f32[n]       one scale per row
"""
from __future__ import annotations

import numpy as np

# Seeds: one generator per tensor so tensors can be regenerated independently.
SEED_X, SEED_WQ, SEED_WS, SEED_WG, SEED_R = 0, 1, 2, 3, 4


def _rng(seed_base: int, which: int, copy: int = 0, layer: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed_base + which + 100 * copy + 1000 * layer))


def _e4m3_positive_finite():
    b = np.arange(1, 0x7F, dtype=np.uint32)          # 0x01 .. 0x7E
    e, m = (b >> 3) & 0xF, (b & 7).astype(np.float64)
    v = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7.0))
    return b.astype(np.uint8), v


def nearest_e4m3(v: np.ndarray) -> np.ndarray:
    """Nearest positive finite E4M3 byte, ties to the even mantissa."""
    bytes_, vals = _e4m3_positive_finite()
    v = np.asarray(v, dtype=np.float64)
    hi = np.clip(np.searchsorted(vals, v), 1, len(vals) - 1)
    lo = hi - 1
    dlo, dhi = v - vals[lo], vals[hi] - v
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((bytes_[hi] & 1) == 0))
    return np.where(pick_hi, bytes_[hi], bytes_[lo]).astype(np.uint8)


def make_x(m: int, k: int, seed_base: int = 0) -> np.ndarray:
    """f16[m,k] ~ N(0,1)."""
    return _rng(seed_base, SEED_X).standard_normal((m, k), dtype=np.float32).astype(np.float16)


def make_weights(n: int, k: int, seed_base: int = 0, copy: int = 0, layer: int = 0):
    """(wq u8[n,k/2], ws u8[n,k/16], wg f32[n]).

    wq: uniform random bytes (all 16 codes, both zeros).  ws: E4M3 bytes of positive finite
    values uniform in log2 over [2^-6, 2^2].  wg: uniform [0.5, 2.0)."""
    if k % 16:
        raise ValueError("k must be a multiple of 16")
    wq = _rng(seed_base, SEED_WQ, copy, layer).integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    u = _rng(seed_base, SEED_WS, copy, layer).uniform(-6.0, 2.0, size=(n, k // 16))
    ws = nearest_e4m3(np.exp2(u))
    wg = _rng(seed_base, SEED_WG, copy, layer).uniform(0.5, 2.0, size=n).astype(np.float32)
    return wq, ws, wg


def make_residual(m: int, n: int, seed_base: int = 0) -> np.ndarray:
    return _rng(seed_base, SEED_R).standard_normal((m, n), dtype=np.float32)


def make_case(m: int, n: int, k: int, seed_base: int = 0):
    x = make_x(m, k, seed_base)
    wq, ws, wg = make_weights(n, k, seed_base)
    return x, wq, ws, wg


def adversarial_dequant_case():
    """Correctness-only weights: every scale byte (subnormals, negatives, the two NaN bytes)
    against every code, with row scales that are tiny, huge, negative, and that make the
    f32 product a rounding tie for the f16 conversion.  Returns (wq, ws, wg) with k = 4096:
    each row holds all 256 scale bytes, each group of 16 columns all 16 codes."""
    gs = [1.0, -1.0, 0.5, 2.0, 1.0 / 3.0, 3.0, 1e-8, 1e-5, 6.1e-5, 1e-3, 17.0, 1e3, 65504.0 / 6.0,
          1e5, 3e38, 1e-38, 1e-45, 0.0, -0.0, np.float32(np.inf), np.float32(np.nan),
          1.0009765625, 1.00048828125, 1.000244140625, 0.99951171875, 1.0 + 2.0 ** -12, 1.0 + 3 * 2.0 ** -12,
          2.0 ** -14, 2.0 ** -15, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25, 2.0 ** -10 + 2.0 ** -22]
    rng = np.random.Generator(np.random.PCG64(77))
    extra = np.concatenate([rng.uniform(0.5, 2.0, 480), np.exp2(rng.uniform(-30, 30, 256)),
                            -np.exp2(rng.uniform(-20, 18, 255))]).astype(np.float32)
    wg = np.concatenate([np.array(gs, dtype=np.float32), extra])
    n = wg.size                                    # 1024 rows
    k = 4096
    ws = np.tile(np.arange(256, dtype=np.uint8), (n, 1))
    codes = np.tile(np.arange(16, dtype=np.uint8), (n, k // 16))
    # rotate the code order per row so every nibble position meets every code
    shift = (np.arange(n) % 16)[:, None]
    codes = (codes + shift) % 16
    wq = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return wq, ws, wg
