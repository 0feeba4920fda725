"""The entry point that allocates no device memory (lexb_gemm_fp4_splitk_static), through the C ABI.

Who needs it: a serving process that reserved the whole device for its own pools at start-up, or a
decode loop that cannot take the stall of an allocation - callers for whom the workspace that
lexb_gemm_fp4_plan allocates for split-K is not an option.  The library's built-in scratch array is
shared by every call and keeps the previous call's contents, so the check is made on two calls in a
row with different inputs: each must equal the planned pipeline's result bit for bit (same kernel, same
split, same order of summation), and both must agree with the oracle to the usual tolerance.
This file sorts last on purpose, so that a run that stops at the first failure has run everything else.
"""
import numpy as np
import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import inputs
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from lex_gpu_b200 import build
    build.build()
    g = L.Gpu(0)
    yield g
    g.close()


def _static(gpu, x, wq, ws, wg, r, splits):
    m, k = x.shape
    n = wq.shape[0]
    q = L.QBuf(gpu, wq, ws, wg)
    xb = gpu.upload(x)
    rb = gpu.upload(r) if r is not None else None
    yb = gpu.alloc(4 * m * n)
    gpu.memset(yb, 0xFF)
    gpu.gemm_fp4_splitk_static(m, n, k, splits, q.bind(xb, rb, yb))
    y = gpu.download(yb, np.float32, (m, n))
    assert gpu.status_word() == 0
    return y


def test_static_scratch_matches_the_planned_pipeline_on_two_calls_in_a_row(gpu):
    # (192 tokens: a tile of one token block; the static entry point and the planner may cut the tokens into
    # different tiles - the sums per element, and so the bits, are the same)
    cases = [(512, 384, 2048, 4, True, 11), (300, 256, 1024, 2, False, 12), (192, 256, 1024, 2, True, 13)]
    for m, n, k, splits, with_r, seed in cases:
        x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=seed)
        r = inputs.make_residual(m, n, seed_base=seed) if with_r else None
        got = _static(gpu, x, wq, ws, wg, r, splits)
        planned = L.gemm_fp4(gpu, x, wq, ws, wg, r=r, kernel=3, k_splits=splits)
        assert np.isfinite(got).all()
        assert np.array_equal(got, planned)
        err, scale, rel = O.err_of_scale(got, O.gemm_fp4(x, wq, ws, wg, r=r))
        assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3


def test_static_scratch_calls_take_no_device_memory(gpu):
    """What the entry point is for: once the first call on the device has resolved the array's address, further
    calls leave the amount of free device memory where it was."""
    import torch
    m, n, k, splits = 512, 256, 1024, 2
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=14)
    q = L.QBuf(gpu, wq, ws, wg)
    xb, yb = gpu.upload(x), gpu.alloc(4 * m * n)
    gpu.gemm_fp4_splitk_static(m, n, k, splits, q.bind(xb, None, yb))        # first call: set-up
    gpu.sync()
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    for _ in range(5):
        gpu.gemm_fp4_splitk_static(m, n, k, splits, q.bind(xb, None, yb))
    gpu.sync()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == before
    err, scale, rel = O.err_of_scale(gpu.download(yb, np.float32, (m, n)), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3


def test_static_scratch_refuses_what_does_not_fit(gpu):
    b = gpu.alloc(1 << 20)
    with pytest.raises(L.LexbError) as e:                       # 8 splits of 2048 x 5120 f32 = 320 MiB
        gpu.gemm_fp4_splitk_static(2048, 5120, 17408, 8, [b, b, b, b, b])
    assert e.value.code == 4 and "scratch" in e.value.message and str(32 << 20) in e.value.message
    with pytest.raises(L.LexbError):
        gpu.gemm_fp4_splitk_static(512, 256, 1024, 1, [b, b, b, b, b])      # one split needs no scratch: not this call
    with pytest.raises(L.LexbError):
        gpu.gemm_fp4_splitk_static(512, 200, 1024, 2, [b, b, b, b, b])      # n % 128
