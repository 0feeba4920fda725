"""The `gemm_fp4` operator over liblexb, in the vocabulary of the reference:
`Gemm` is lex_msl::gemm::Gemm (crates/lex-msl/src/gemm.rs:40-57), `QBuf` the packed weight
triple with its positional binding (crates/lex-rt/src/qwen_run.rs:375-387), and
`GemmKernels.get` the per-shape selector lx_kernels::gemm (crates/lex-rt/src/lx_kernels.rs:43-107).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .device import Buffer, Gpu, Pipeline


@dataclass(frozen=True)
class Gemm:
    m: int
    n: int
    k: int
    residual: bool = False

    def flops(self) -> float:
        """2 m n k, as crates/lex-rt/examples/gemm_bench.rs:162 counts."""
        return 2.0 * self.m * self.n * self.k

    def weight_bytes(self) -> int:
        """Codes + group scales + row scales: n k/2 + n k/16 + 4 n."""
        return self.n * self.k // 2 + self.n * self.k // 16 + 4 * self.n

    def total_bytes(self) -> int:
        return self.weight_bytes() + 2 * self.m * self.k + 4 * self.m * self.n * (2 if self.residual else 1)


class QBuf:
    """Resident NVFP4 weights of one matrix: wq u8[n,k/2], ws u8[n,k/16], wg f32[n]."""

    def __init__(self, gpu: Gpu, wq: np.ndarray, ws: np.ndarray, wg: np.ndarray):
        n, kh = wq.shape
        if ws.shape != (n, kh // 8) or wg.shape != (n,):
            raise ValueError(f"weight shapes do not fit: wq{wq.shape} ws{ws.shape} wg{wg.shape}")
        self.n, self.k = n, 2 * kh
        self.wq = gpu.upload(np.ascontiguousarray(wq).view(np.uint8))
        self.ws = gpu.upload(np.ascontiguousarray(ws).view(np.uint8))
        self.wg = gpu.upload(np.ascontiguousarray(wg, dtype=np.float32))

    def bind(self, x: Buffer, r: Optional[Buffer], y: Buffer) -> list[Buffer]:
        """[x, wq, ws, wg, (r), y]"""
        return [x, self.wq, self.ws, self.wg] + ([r] if r is not None else []) + [y]

    @classmethod
    def gate_up(cls, gpu: Gpu, gate: "QBuf", up: "QBuf") -> "QBuf":
        """The weights of gate and up with their rows interleaved on the device (row 2j = gate j, 2j + 1 = up j):
        what the fused launch Gpu.run_silu multiplies by.  A load-time step."""
        if (gate.n, gate.k) != (up.n, up.k):
            raise ValueError("gate and up differ in shape")
        q = cls.__new__(cls)
        q.n, q.k = 2 * gate.n, gate.k
        q.wq, q.ws, q.wg = gpu.alloc(q.n * q.k // 2), gpu.alloc(q.n * q.k // 16), gpu.alloc(q.n * 4)
        gpu.interleave_rows(gate.wq, up.wq, gate.n, gate.k // 2, q.wq)
        gpu.interleave_rows(gate.ws, up.ws, gate.n, gate.k // 16, q.ws)
        gpu.interleave_rows(gate.wg, up.wg, gate.n, 4, q.wg)
        gpu.sync()
        return q

    def close(self) -> None:
        for b in (self.wq, self.ws, self.wg):
            b.close()


class GemmKernels:
    """One planned pipeline per (m, n, k, residual), built on first use."""

    def __init__(self, gpu: Gpu):
        self.gpu = gpu
        self._cache: dict[tuple, Pipeline] = {}

    def get(self, g: Gemm, **sched) -> Pipeline:
        key = (g, tuple(sorted(sched.items())))
        if key not in self._cache:
            self._cache[key] = self.gpu.plan_gemm_fp4(g.m, g.n, g.k, g.residual, **sched)
        return self._cache[key]


def gemm_fp4(gpu: Gpu, x: np.ndarray, wq: np.ndarray, ws: np.ndarray, wg: np.ndarray,
             r: Optional[np.ndarray] = None, **sched) -> np.ndarray:
    """Host arrays in, host array out: upload, one launch, download.  For tests and examples;
    a runtime keeps QBufs resident and calls Gpu.run / Gpu.run_host per step."""
    m, k = x.shape
    n = wq.shape[0]
    if x.dtype != np.float16:
        raise TypeError("x must be float16")
    pipe = gpu.plan_gemm_fp4(m, n, k, r is not None, **sched)
    q = QBuf(gpu, wq, ws, wg)
    xb = gpu.upload(x)
    rb = gpu.upload(np.ascontiguousarray(r, dtype=np.float32)) if r is not None else None
    yb = gpu.alloc(4 * m * n)
    gpu.memset(yb, 0xFF)                      # NaN pattern: every element must be written
    try:
        gpu.run(pipe, q.bind(xb, rb, yb))
        y = gpu.download(yb, np.float32, (m, n))
        st = gpu.status_word()
        if st:
            raise RuntimeError(f"gemm_fp4 kernel reported status 0x{st:x}")
        return y
    finally:
        for b in (xb, yb, rb):
            if b is not None:
                b.close()
        q.close()
        pipe.close()


def matmul_fp4(gpu: Gpu, x: np.ndarray, wq: np.ndarray, ws: np.ndarray, wg: np.ndarray,
               r: Optional[np.ndarray] = None, **sched) -> np.ndarray:
    """matmul_q_x with the NVFP4 layout, host arrays in and out (llama.rs:444-499): t <= 32 tokens of f16 or
    f32 activations against weights used as f32 (not rounded to f16).  For tests and examples."""
    m, k = x.shape
    n = wq.shape[0]
    if x.dtype not in (np.float16, np.float32):
        raise TypeError("x must be float16 (x_half) or float32")
    pipe = gpu.plan_matmul_fp4(m, n, k, r is not None, x.dtype == np.float16, **sched)
    q = QBuf(gpu, wq, ws, wg)
    xb = gpu.upload(x)
    rb = gpu.upload(np.ascontiguousarray(r, dtype=np.float32)) if r is not None else None
    yb = gpu.alloc(4 * m * n)
    gpu.memset(yb, 0xEE)                      # a finite, absurd pattern (NaN is a legal result here)
    try:
        gpu.run(pipe, q.bind(xb, rb, yb))
        y = gpu.download(yb, np.float32, (m, n))
        st = gpu.status_word()
        if st:
            raise RuntimeError(f"matmul_fp4 kernel reported status 0x{st:x}")
        return y
    finally:
        for b in (xb, yb, rb):
            if b is not None:
                b.close()
        q.close()
        pipe.close()


def dequant_fp4_f16(gpu: Gpu, wq: np.ndarray, ws: np.ndarray, wg: np.ndarray) -> np.ndarray:
    """uint16 [n,k]: the f16 bit patterns the kernels multiply by."""
    n, kh = wq.shape
    k = 2 * kh
    q = QBuf(gpu, wq, ws, wg)
    out = gpu.alloc(2 * n * k)
    try:
        gpu.dequant_fp4_f16(n, k, q.wq, q.ws, q.wg, out)
        return gpu.download(out, np.uint16, (n, k))
    finally:
        out.close()
        q.close()
