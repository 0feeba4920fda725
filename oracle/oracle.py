"""Python face of the CPU oracle for `gemm_fp4`.

TEST INFRASTRUCTURE ONLY: imported by tests, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

Three independent statements of the same arithmetic live here so that they can be
checked against one another:

* the C library built from ``gemm_fp4_ref.c`` (follows the reference interpreter,
  crates/lex-front/src/interp.rs:30-47, 76-82, 500-526, 643-657),
* a numpy twin (``np_*``) that uses numpy's own float16/float32 casts, and
* the f64 restatement the reference's own test uses as its expected value
  (crates/lex-front/tests/syntax.rs:509-523, 559-571).

Parity status: pinned against the reference's known-answer recipes; the f16 bit
patterns of staged weights are "parity unpinned" by any reference fixture (they
follow from IEEE round-to-nearest-even alone).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None

# Decode tables written out as literals: the values of interp.rs:31 and the OCP
# e4m3fn format, stated a second time (as scripts/qwen_nvfp4.py:27-42 does).
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                 -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def e4m3_table() -> np.ndarray:
    b = np.arange(256, dtype=np.uint32)
    e = (b >> 3) & 0xF
    m = (b & 7).astype(np.float64)
    v = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7.0))
    v = np.where((e == 15) & ((b & 7) == 7), np.nan, v)
    v = np.where(b >> 7 == 1, -v, v)
    return v.astype(np.float32)


E4M3 = e4m3_table()


def build(force: bool = False) -> Path:
    """Compile the C oracle beside its source (make; gcc with OpenMP)."""
    so = HERE / "liblexoracle.so"
    src = HERE / "gemm_fp4_ref.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(str(build()))
        u32, vp, ci = ctypes.c_uint32, ctypes.c_void_p, ctypes.c_int
        L.lexo_e2m1.restype = ctypes.c_float
        L.lexo_e2m1.argtypes = [ctypes.c_uint8]
        L.lexo_e4m3.restype = ctypes.c_float
        L.lexo_e4m3.argtypes = [ctypes.c_uint8]
        L.lexo_f32_to_f16.restype = ctypes.c_uint16
        L.lexo_f32_to_f16.argtypes = [ctypes.c_float]
        L.lexo_f16_to_f32.restype = ctypes.c_float
        L.lexo_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.lexo_dequant_fp4_f16.restype = None
        L.lexo_dequant_fp4_f16.argtypes = [u32, u32, vp, vp, vp, vp]
        L.lexo_gemm_fp4_rows.restype = ci
        L.lexo_gemm_fp4_rows.argtypes = [u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, u32, u32, ci]
        L.lexo_matmul_q_x.restype = ci
        L.lexo_matmul_q_x.argtypes = [u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, ci]
        L.lexo_max_rel_err.restype = ctypes.c_float
        L.lexo_max_rel_err.argtypes = [vp, vp, ctypes.c_size_t]
        L.lexo_err_of_scale.restype = None
        L.lexo_err_of_scale.argtypes = [vp, vp, ctypes.c_size_t, vp]
        L.lexo_max_threads.restype = ci
        _LIB = L
    return _LIB


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _check_shapes(x16, wq, ws, wg):
    m, k = x16.shape
    n = wq.shape[0]
    if x16.dtype != np.float16 and x16.dtype != np.uint16:
        raise TypeError("x must be float16 (or its uint16 bit patterns)")
    if wq.shape != (n, k // 2) or ws.shape != (n, k // 16) or wg.shape != (n,):
        # the rank-1 row-scale rule of crates/lex-front/tests/tensor_shapes.rs:65-67
        raise ValueError(f"shapes do not fit gemm_fp4: x{x16.shape} wq{wq.shape} ws{ws.shape} wg{wg.shape}")
    return m, n, k


def gemm_fp4(x16, wq, ws, wg, r=None, bk: int = 64, rows=None, threads: int = 0) -> np.ndarray:
    """The oracle: y f32[m,n].  `rows=(n0,n1)` computes only those W rows (others stay 0)."""
    m, n, k = _check_shapes(x16, wq, ws, wg)
    x16 = np.ascontiguousarray(x16).view(np.uint16)
    wq = np.ascontiguousarray(wq).view(np.uint8)
    ws = np.ascontiguousarray(ws).view(np.uint8)
    wg = np.ascontiguousarray(wg, dtype=np.float32)
    y = np.zeros((m, n), dtype=np.float32)
    rp = None
    if r is not None:
        r = np.ascontiguousarray(r, dtype=np.float32)
        assert r.shape == (m, n)
        rp = _p(r)
    n0, n1 = rows if rows is not None else (0, n)
    rc = lib().lexo_gemm_fp4_rows(m, n, k, bk, _p(x16), _p(wq), _p(ws), _p(wg), rp, _p(y), n0, n1, threads)
    if rc != 0:
        raise ValueError(f"gemm_fp4 oracle rejected the shape (rc={rc}): k={k} does not divide by bk={bk}")
    return y


def matmul_q_x(x, wq, ws, wg, r=None, kc: int = 0, threads: int = 0) -> np.ndarray:
    """matmul_q_x with the NVFP4 layout (crates/lex-front/src/llama.rs:444-499): y f32[t, n_out] with the
    weights as f32 (not rounded to f16) and a sequential f32 sum per chunk of kc columns (kc = 0: the
    whole row, as the runtime calls it).  x is float16 or float32 [t, n_in]."""
    x = np.asarray(x)
    if x.dtype not in (np.float16, np.float32):
        raise TypeError("x must be float16 or float32")
    m, k = x.shape
    n = wq.shape[0]
    if wq.shape != (n, k // 2) or ws.shape != (n, k // 16) or wg.shape != (n,):
        raise ValueError(f"shapes do not fit matmul_q_x: x{x.shape} wq{wq.shape} ws{ws.shape} wg{wg.shape}")
    xf = np.ascontiguousarray(x.astype(np.float32))
    wq = np.ascontiguousarray(wq).view(np.uint8)
    ws = np.ascontiguousarray(ws).view(np.uint8)
    wg = np.ascontiguousarray(wg, dtype=np.float32)
    y = np.zeros((m, n), dtype=np.float32)
    rp = None
    if r is not None:
        r = np.ascontiguousarray(r, dtype=np.float32)
        assert r.shape == (m, n)
        rp = _p(r)
    rc = lib().lexo_matmul_q_x(m, n, k, kc or k, _p(xf), _p(wq), _p(ws), _p(wg), rp, _p(y), threads)
    if rc != 0:
        raise ValueError(f"matmul_q_x oracle rejected the shape (rc={rc}): kc={kc or k} must divide k={k} in groups of 16")
    return y


def dequant_fp4_f16(wq, ws, wg) -> np.ndarray:
    """uint16 [n,k]: the f16 bit pattern of every staged weight."""
    n, kh = wq.shape
    k = 2 * kh
    wq = np.ascontiguousarray(wq).view(np.uint8)
    ws = np.ascontiguousarray(ws).view(np.uint8)
    wg = np.ascontiguousarray(wg, dtype=np.float32)
    out = np.empty((n, k), dtype=np.uint16)
    lib().lexo_dequant_fp4_f16(n, k, _p(wq), _p(ws), _p(wg), _p(out))
    return out


def max_rel_err(got, want) -> float:
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    return float(lib().lexo_max_rel_err(_p(got), _p(want), got.size))


def err_of_scale(got, want):
    """(error of scale, scale, floored per-element relative error)."""
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    out = np.zeros(3, dtype=np.float64)
    lib().lexo_err_of_scale(_p(got), _p(want), got.size, _p(out))
    return float(out[0]), float(out[1]), float(out[2])


def max_threads() -> int:
    return int(lib().lexo_max_threads())


# ---------------------------------------------------------------- numpy twin

def np_codes(wq: np.ndarray) -> np.ndarray:
    """uint8 [n,k]: the 4-bit code of every column; even column = low nibble (interp.rs:650)."""
    b = wq.view(np.uint8)
    out = np.empty((b.shape[0], b.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = b & 0xF
    out[:, 1::2] = b >> 4
    return out


def np_dequant_f32(wq, ws, wg) -> np.ndarray:
    """f32 [n,k] before staging: (e2m1 * e4m3) * wg, each product rounded to f32."""
    with np.errstate(invalid="ignore", over="ignore"):
        v = E2M1[np_codes(wq)] * np.repeat(E4M3[ws.view(np.uint8)], 16, axis=1)
        return (v * wg.astype(np.float32)[:, None]).astype(np.float32)


def np_dequant_f16(wq, ws, wg) -> np.ndarray:
    with np.errstate(over="ignore", invalid="ignore"):
        return np_dequant_f32(wq, ws, wg).astype(np.float16)


def np_gemm_fp4(x16, wq, ws, wg, r=None, bk: int = 64) -> np.ndarray:
    """Small cases only: the interpreter's order, vectorised across (i, j)."""
    m, n, k = _check_shapes(x16, wq, ws, wg)
    if k % bk:
        raise ValueError("k does not divide by bk")
    a = x16.view(np.float16).astype(np.float32)
    b = np_dequant_f16(wq, ws, wg).astype(np.float32)
    acc = np.zeros((m, n), dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        for t in range(0, k, bk):
            s = np.zeros((m, n), dtype=np.float32)
            for p in range(t, t + bk):
                s = s + a[:, p, None] * b[None, :, p]
            acc = acc + s
        if r is not None:
            acc = acc + r.astype(np.float32)
    return acc


# ------------------------------------------- the reference's own test recipes

def lcg_fill(length: int, seed: int) -> np.ndarray:
    """crates/lex-front/tests/syntax.rs:387-395: floats in [-0.5, 0.5)."""
    out = np.empty(length, dtype=np.float32)
    x = seed & 0xFFFFFFFF
    for i in range(length):
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(x >> 9) / np.float32(1 << 23)) - np.float32(0.5)
    return out


def kat_inputs(m: int, n: int, k: int, residual: bool = False):
    """Inputs of `the_fp4_gemm_decodes_stages_and_multiplies` (syntax.rs:543-551) or, with
    `residual`, of `the_residual_epilogue_adds_the_stream_to_the_product` (syntax.rs:652-658)."""
    if not residual:
        x = lcg_fill(m * k, 31)
        i = np.arange(n * k // 2, dtype=np.int64)
        q = ((i * 97 + 13) % 256).astype(np.uint8)
        j = np.arange(n * k // 16, dtype=np.int64)
        sc = (0x30 + j % 7).astype(np.uint8)
        g = (0.5 + (np.arange(n) % 5).astype(np.float32) * np.float32(0.25)).astype(np.float32)
        r = None
    else:
        x = lcg_fill(m * k, 51)
        i = np.arange(n * k // 2, dtype=np.int64)
        q = ((i * 31 + 7) % 256).astype(np.uint8)
        j = np.arange(n * k // 16, dtype=np.int64)
        sc = (0x30 + j % 5).astype(np.uint8)
        g = (0.5 + (np.arange(n) % 3).astype(np.float32) * np.float32(0.5)).astype(np.float32)
        r = lcg_fill(m * n, 52).reshape(m, n)
    # Tensor::new rounds x to f16 on creation (interp.rs:61-69).
    x16 = x.reshape(m, k).astype(np.float16)
    return x16, q.reshape(n, k // 2), sc.reshape(n, k // 16), g, r


def ref_fill(length: int, seed: int) -> np.ndarray:
    """The input recipe of the reference's GPU tests (crates/lex-cuda/tests/device_gpu.rs:29-36):
    x_i = ((i * 2654435761 + seed) mod 2^32 >> 9) / 2^22 - 1, in [-1, 1)."""
    i = np.arange(length, dtype=np.uint64)
    x = (i * np.uint64(2654435761) + np.uint64(seed)) & np.uint64(0xFFFFFFFF)
    return ((x >> np.uint64(9)).astype(np.float32) / np.float32(4194304.0)) - np.float32(1.0)


def ref_nvfp4_bytes(n_out: int, n_in: int, mul: int, add: int, scale_base: int, scale_mod: int):
    """Codes and scale bytes as those tests build them (device_gpu.rs:138-143, 163-168, 189-194, 255-260):
    code byte i = (i * mul + add) & 0xFF and scale byte i = scale_base + i % scale_mod, each minus 128 as an
    i8 VALUE - so the byte the kernels see has bit 7 flipped (scale bytes come out with the sign bit set:
    negative scales)."""
    i = np.arange(n_out * n_in // 2, dtype=np.uint64)
    codes = ((((i * np.uint64(mul) + np.uint64(add)) & np.uint64(0xFF)).astype(np.int64) - 128) & 0xFF).astype(np.uint8)
    j = np.arange(n_out * n_in // 16, dtype=np.int64)
    scales = ((scale_base + j % scale_mod - 128) & 0xFF).astype(np.uint8)
    return codes.reshape(n_out, n_in // 2), scales.reshape(n_out, n_in // 16)


def f64_restatement(x16, wq, ws, wg) -> np.ndarray:
    """The expected value of syntax.rs:559-575: decode in f64 with the test's own tables,
    round the weight to f16 from f64, multiply and sum in f64."""
    mag = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float64)
    c = np_codes(wq)
    e2 = np.where(c & 8, -mag[c & 7], mag[c & 7])
    b = ws.view(np.uint8).astype(np.int64)
    e, mm = (b >> 3) & 15, (b & 7).astype(np.float64)
    v = np.where(e == 0, mm / 8.0 * 2.0 ** -6, (1.0 + mm / 8.0) * 2.0 ** (e.astype(np.float64) - 7.0))
    v = np.where(b & 0x80, -v, v)
    w = e2 * np.repeat(v, 16, axis=1) * wg.astype(np.float64)[:, None]
    w = w.astype(np.float16).astype(np.float64)          # half::f16::from_f64
    return x16.view(np.float16).astype(np.float64) @ w.T


def np_silu_mul(g: np.ndarray, u: np.ndarray, out_f16: bool = False) -> np.ndarray:
    """silu(g) * u as the interpreter evaluates lex_front::llama::silu_mul (crates/lex-front/src/llama.rs:879-888,
    sigmoid = 1 / (1 + exp(-x)), crates/lex-front/src/ir.rs:244): f32 throughout, one rounding per operation,
    then the optional conversion to f16."""
    g = g.astype(np.float32)
    u = u.astype(np.float32)
    one = np.float32(1.0)
    with np.errstate(over="ignore"):
        sg = one / (one + np.exp(-g, dtype=np.float32))
        y = (g * sg) * u
    return y.astype(np.float16) if out_f16 else y


def ensure_built() -> None:
    build()
    if not os.path.exists(HERE / "liblexoracle.so"):
        raise RuntimeError("oracle library missing after build")


# ------------------------------------------- the integer-activation path (crates/lex-msl/src/int8.rs)

def np_quant16(x: np.ndarray):
    """quant16 (crates/lex-msl/src/int8.rs:47-114) restated in numpy float32, operation for operation: per group
    of 16 values the largest magnitude mx, inv = 32767 / mx (0 for a group of zeros), q = rint(v * inv) as int16
    (round half to even, as __float2int_rn), scale mx / 32767.  Returns (xq int16 [m, k], xs float32 [m, k/16])."""
    x = np.asarray(x)
    m, k = x.shape
    if k % 32:
        raise ValueError("quant16: inputs are not whole groups of 32")
    v = x.astype(np.float32).reshape(m, k // 16, 16)
    mx = np.abs(v).max(axis=2)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(mx > 0, np.float32(32767.0) / mx, np.float32(0.0)).astype(np.float32)
    q = np.rint((v * inv[:, :, None]).astype(np.float32)).astype(np.int32)
    xq = (q & 0xFFFF).astype(np.uint16).view(np.int16).reshape(m, k)
    xs = (mx / np.float32(32767.0)).astype(np.float32)
    return xq, xs


def np_matmul_int8_f64(xq, xs, wq, ws, wg, r=None) -> np.ndarray:
    """What matmul_int8 computes (crates/lex-msl/src/int8.rs:121-223) in f64: per group of 16 the integer dot product
    of the int16 activations with twice the E2M1 values, times the group's weight scale and activation scale, summed
    over the row, times the row scale and one half, plus the residual.  (The kernel adds the groups in f32 in a
    lane-strided order; this is its value without those roundings.)"""
    m, k = xq.shape
    c = np_codes(wq)
    e = E2M1[c].astype(np.float64)                                    # [n, k]
    s = np.repeat(E4M3[ws.view(np.uint8)].astype(np.float64), 16, axis=1)
    xv = xq.astype(np.float64) * np.repeat(xs.astype(np.float64), 16, axis=1)
    y = (xv @ (e * s).T) * wg.astype(np.float64)[None, :]
    if r is not None:
        y = y + r.astype(np.float64)
    return y
