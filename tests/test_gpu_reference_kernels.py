"""The reference's own CUDA kernels, compiled for sm_100a, run beside this library and the CPU oracle.

The reference cannot be built as a whole here (Rust), but two of its kernels exist as CUDA text in its tree
and are compiled from there by oracle/build_ref.py: the emitted decode matvec `matvec_nvfp4_17408x5120`
(crates/lex-msl/tests/golden/matvec_nvfp4_17408x5120_cuda.cu) and instances of the hand-scheduled GEMM
(crates/lex-msl/src/gemm.rs:89-320).  These tests hold three parties to one another on the same inputs:

    reference kernel  <->  CPU oracle      (pins the oracle to outputs of the reference's own code)
    reference kernel  <->  this library    (the drop-in claim)

at the reference's own bars for these pairs: 1e-4 of scale for the matvec against the interpreter
(crates/lex-cuda/tests/device_gpu.rs:130-204) and 2e-3 of scale for the GEMM against the interpreter
(crates/lex-cuda/tests/device_gpu.rs:210-305).  The GEMM kernel folds the group scale into the row scale
before it multiplies (crates/lex-msl/src/gemm.rs:254-255), so its weights differ from the interpreter's by one
f16 step in about one weight in 10^5; that is inside the bar and is why the bar is not zero.
"""
import numpy as np
import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import inputs
from oracle import oracle as O
from oracle import refkernels as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from lex_gpu_b200 import build
    build.build()
    g = L.Gpu(0)
    yield g
    g.close()


def of_scale(got, want):
    assert np.isfinite(got).all(), "non-finite output (an element was not written?)"
    err, scale, rel = O.err_of_scale(got, want)
    assert scale > 1e-3, "the reference output is all but zero"
    return err, rel


def need(entry):
    if not R.available(entry):
        pytest.fail(f"oracle/_ref/{entry}.so is missing: run `python oracle/build_ref.py` where the reference tree is present")


# ---------------------------------------------------------------- the emitted decode matvec (f32 x)

def matvec_cases():
    # the reference's own recipe for the 5120-wide matvec (crates/lex-cuda/tests/device_gpu.rs:161-182: LCG
    # activations seed 9, code bytes (i*131+17)&0xff and scale bytes 0x30 + i%11 as i8 values minus 128, row
    # scales 0.5 + (i%3)/4), at the golden kernel's shape
    x = O.ref_fill(5120, 9).reshape(1, 5120)
    wq, ws = O.ref_nvfp4_bytes(17408, 5120, 131, 17, 0x30, 11)
    wg = (0.5 + (np.arange(17408) % 3).astype(np.float32) * np.float32(0.25)).astype(np.float32)
    yield "reference recipe", x, wq, ws, wg
    # the benchmark's seeded distributions, x kept in f32
    wq, ws, wg = inputs.make_weights(17408, 5120)
    x = np.random.Generator(np.random.PCG64(0)).standard_normal((1, 5120), dtype=np.float32)
    yield "benchmark distribution", x, wq, ws, wg


def test_reference_matvec_kernel_pins_the_oracle_and_the_library(gpu):
    need(R.MATVEC_ENTRY)
    for name, x, wq, ws, wg in matvec_cases():
        ref = R.matvec(x, wq, ws, wg)
        want = O.matmul_q_x(x, wq, ws, wg)
        e_oracle, _ = of_scale(want, ref)
        got = L.matmul_fp4(gpu, x, wq, ws, wg)
        e_lib, _ = of_scale(got, ref)
        print(f"  {name}: oracle vs reference kernel {e_oracle:.2e}, library vs reference kernel {e_lib:.2e} of scale")
        assert e_oracle <= 1e-4 and e_lib <= 1e-4


# ---------------------------------------------------------------- the hand-scheduled GEMM (f16 x)

GEMM_CASES = [(256, 512, 1024, False), (96, 256, 1024, True), (17, 128, 256, False), (40, 128, 512, False)]


@pytest.mark.parametrize("m,n,k,residual", GEMM_CASES)
def test_reference_gemm_kernel_small_and_ragged(gpu, m, n, k, residual):
    need(R.gemm_entry(m, n, k, residual))
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=m + n + k)
    r = inputs.make_residual(m, n, seed_base=m) if residual else None
    ref = R.gemm(x, wq, ws, wg, r)
    e_oracle, _ = of_scale(O.gemm_fp4(x, wq, ws, wg, r=r), ref)
    e_lib, _ = of_scale(L.gemm_fp4(gpu, x, wq, ws, wg, r=r), ref)
    print(f"  oracle vs reference kernel {e_oracle:.2e}, library vs reference kernel {e_lib:.2e} of scale")
    assert e_oracle <= 2e-3 and e_lib <= 2e-3


def test_reference_gemm_kernel_with_the_reference_tests_recipe(gpu):
    """Inputs as crates/lex-cuda/tests/device_gpu.rs:255-270 builds them: activations fill(seed 3) rounded to f16,
    code bytes (i*97+3)&0xff and scale bytes 0x34 + i%7 as i8 values minus 128 (negative scales), row scales
    0.5 + (i%5)/8, residual fill(seed 11)."""
    m, n, k = 96, 256, 1024
    need(R.gemm_entry(m, n, k, True))
    x = O.ref_fill(m * k, 3).reshape(m, k).astype(np.float16)
    wq, ws = O.ref_nvfp4_bytes(n, k, 97, 3, 0x34, 7)
    wg = (0.5 + (np.arange(n) % 5).astype(np.float32) * np.float32(0.125)).astype(np.float32)
    r = O.ref_fill(m * n, 11).reshape(m, n)
    ref = R.gemm(x, wq, ws, wg, r)
    e_oracle, _ = of_scale(O.gemm_fp4(x, wq, ws, wg, r=r), ref)
    e_lib, _ = of_scale(L.gemm_fp4(gpu, x, wq, ws, wg, r=r), ref)
    print(f"  oracle vs reference kernel {e_oracle:.2e}, library vs reference kernel {e_lib:.2e} of scale")
    assert e_oracle <= 2e-3 and e_lib <= 2e-3


@pytest.mark.parametrize("n,k,residual", [(17408, 5120, False), (5120, 17408, True)])
def test_reference_gemm_kernel_headline_shapes(gpu, n, k, residual):
    """m = 512 at the 27B MLP shapes: the library against the reference's kernel over the whole output, the
    oracle against it on a slice of rows."""
    m = 512
    need(R.gemm_entry(m, n, k, residual))
    x, wq, ws, wg = inputs.make_case(m, n, k)
    r = inputs.make_residual(m, n) if residual else None
    ref = R.gemm(x, wq, ws, wg, r)
    got = L.gemm_fp4(gpu, x, wq, ws, wg, r=r)
    e_lib, rel_lib = of_scale(got, ref)
    lo, hi = n // 2 - 128, n // 2 + 128
    want = O.gemm_fp4(x, wq, ws, wg, r=r, rows=(lo, hi))
    e_oracle, _ = of_scale(want[:, lo:hi], ref[:, lo:hi])
    print(f"  oracle vs reference kernel {e_oracle:.2e} (rows {lo}..{hi}), library vs reference kernel {e_lib:.2e} of scale "
          f"({rel_lib:.2e} per element)")
    assert e_oracle <= 2e-3 and e_lib <= 2e-3
