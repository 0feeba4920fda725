"""Error paths of the C ABI, reached by failures made on the host.

lexb_debug_fail_next arms a site (device allocation, host<->device copy, kernel launch, tensor-map encoding) so
that the nth call reaching it reports a CUDA error instead of being made - the counterpart of handing the
reference's backend a driver table whose entries fail (the `api!` table, crates/lex-cuda/src/device.rs:88-132).
Nothing on the device fails, traps or hangs.  Each case checks that the entry point returns LEXB_ERR_CUDA with
a message, that the device memory it had taken is back (cudaMemGetInfo), and that the next ordinary call on
the same handle passes parity.
"""
import numpy as np
import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import device as D, inputs
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ERR_CUDA = 3


@pytest.fixture(scope="module")
def gpu():
    from lex_gpu_b200 import build
    build.build()
    g = L.Gpu(0)
    yield g
    D.debug_fail_next(0)
    g.close()


def free_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def parity_still_holds(gpu, m=64, n=256, k=1024, seed=3):
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=seed)
    err, scale, rel = O.err_of_scale(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3
    assert gpu.status_word() == 0


def test_allocation_failure_in_alloc_and_in_plan(gpu):
    D.debug_fail_next(D.SITE_ALLOC)
    with pytest.raises(L.LexbError) as e:
        gpu.alloc(1 << 20)
    assert e.value.code == ERR_CUDA and "injected" in e.value.message
    gpu.alloc(1 << 20).close()                                   # the site is disarmed after it fired
    before = free_bytes()
    # the split-K workspace of the two-CTA GEMM
    D.debug_fail_next(D.SITE_ALLOC)
    with pytest.raises(L.LexbError) as e:
        gpu.plan_gemm_fp4(512, 5120, 17408)
    assert e.value.code == ERR_CUDA and "workspace" in e.value.message
    # the block-scaled kernel's plan allocates twice (partial products, then digit rows): fail the second
    D.debug_fail_next(D.SITE_ALLOC, nth=2)
    with pytest.raises(L.LexbError) as e:
        gpu.plan_matmul_fp4(8, 1024, 4096, k_splits=2)
    assert e.value.code == ERR_CUDA and "digit-row" in e.value.message
    assert free_bytes() == before                                # the first allocation was given back
    p = gpu.plan_gemm_fp4(512, 5120, 17408)
    assert p.describe().scratch_bytes > 0
    p.close()
    parity_still_holds(gpu)


def test_copy_failure_in_upload_download_and_the_host_call(gpu):
    m, n, k = 64, 256, 512
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=8)
    buf = gpu.alloc(x.nbytes)
    D.debug_fail_next(D.SITE_COPY)
    with pytest.raises(L.LexbError) as e:
        gpu.write(buf, 0, x)
    assert e.value.code == ERR_CUDA and "injected" in e.value.message
    gpu.write(buf, 0, x)
    D.debug_fail_next(D.SITE_COPY)
    with pytest.raises(L.LexbError):
        gpu.download(buf, np.float16, (m, k))
    assert np.array_equal(gpu.download(buf, np.float16, (m, k)), x)
    # lexb_gemm_fp4_run_host: the copy in, then the copy back
    q = L.QBuf(gpu, wq, ws, wg)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    hx, hy = L.HostBuffer(x.nbytes), L.HostBuffer(m * n * 4)
    hx.array(np.float16, (m, k))[:] = x
    xd, yd = gpu.alloc(x.nbytes), gpu.alloc(m * n * 4)
    for nth in (1, 2):
        D.debug_fail_next(D.SITE_COPY, nth=nth)
        with pytest.raises(L.LexbError) as e:
            gpu.run_host(pipe, hx.ptr, xd, q.wq, q.ws, q.wg, None, yd, hy.ptr)
        assert e.value.code == ERR_CUDA
        gpu.sync()
    gpu.run_host(pipe, hx.ptr, xd, q.wq, q.ws, q.wg, None, yd, hy.ptr)
    err, scale, rel = O.err_of_scale(hy.array(np.float32, (m, n)).copy(), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3
    assert gpu.status_word() == 0


@pytest.mark.parametrize("m,n,k,splits", [(4, 256, 1024, 0), (64, 256, 1024, 0), (512, 256, 2048, 2)])
def test_launch_failure_in_every_gemm_fp4_kernel(gpu, m, n, k, splits):
    """Matvec, two-CTA GEMM, and the two-CTA GEMM with its reduction launch (the second launch fails)."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=m)
    q = L.QBuf(gpu, wq, ws, wg)
    xb, yb = gpu.upload(x), gpu.alloc(4 * m * n)
    pipe = gpu.plan_gemm_fp4(m, n, k, k_splits=splits)
    for nth in ((1, 2) if splits else (1,)):
        D.debug_fail_next(D.SITE_LAUNCH, nth=nth)
        with pytest.raises(L.LexbError) as e:
            gpu.run(pipe, q.bind(xb, None, yb))
        assert e.value.code == ERR_CUDA and "injected" in e.value.message
        gpu.sync()
    gpu.memset(yb, 0xFF)
    gpu.run(pipe, q.bind(xb, None, yb))
    err, scale, rel = O.err_of_scale(gpu.download(yb, np.float32, (m, n)), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3
    assert gpu.status_word() == 0


def test_launch_failure_inside_a_step_list(gpu):
    """A list of block-scaled steps that would run as one persistent kernel: the failing launch ends the call
    with an error, and the same list runs afterwards."""
    m, n, k = 2, 1024, 2048
    x = inputs.make_x(m, k, seed_base=21)
    sets = [inputs.make_weights(n, k, seed_base=22, copy=c) for c in range(3)]
    qs = [L.QBuf(gpu, *w) for w in sets]
    xb = gpu.upload(x)
    ys = [gpu.alloc(4 * m * n) for _ in sets]
    pipe = gpu.plan_matmul_fp4(m, n, k, k_splits=1)
    steps = [(pipe, q.bind(xb, None, y)) for q, y in zip(qs, ys)]
    before = free_bytes()
    gpu.run_launches(steps)                                       # (the run's job table is allocated and kept here)
    kept = before - free_bytes()
    D.debug_fail_next(D.SITE_LAUNCH)
    with pytest.raises(L.LexbError) as e:
        gpu.run_launches(steps)
    assert e.value.code == ERR_CUDA
    gpu.sync()
    gpu.run_launches(steps)
    assert before - free_bytes() == kept                          # nothing more was taken by the failed call
    for w, y in zip(sets, ys):
        err, scale, _ = O.err_of_scale(gpu.download(y, np.float32, (m, n)), O.matmul_q_x(x, *w))
        assert scale > 1e-3 and err <= 1e-4
    assert gpu.status_word() == 0


def test_tensor_map_encoding_failure(gpu):
    m, n, k = 300, 256, 1024
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=31)
    q = L.QBuf(gpu, wq, ws, wg)
    xb, yb = gpu.upload(x), gpu.alloc(4 * m * n)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    for nth in (1, 2, 3):                                         # the maps of x, wq and ws
        D.debug_fail_next(D.SITE_ENCODE, nth=nth)
        with pytest.raises(L.LexbError) as e:
            gpu.run(pipe, q.bind(xb, None, yb))
        assert e.value.code == ERR_CUDA and "cuTensorMapEncodeTiled" in e.value.message
    gpu.memset(yb, 0xFF)
    gpu.run(pipe, q.bind(xb, None, yb))                           # nothing half-made was cached
    err, scale, rel = O.err_of_scale(gpu.download(yb, np.float32, (m, n)), O.gemm_fp4(x, wq, ws, wg))
    assert scale > 1e-3 and err <= 2e-3 and rel <= 2e-3
    assert gpu.status_word() == 0


def test_disarming_and_argument_checks(gpu):
    D.debug_fail_next(D.SITE_ALLOC, nth=5)
    D.debug_fail_next(0)
    for _ in range(6):
        gpu.alloc(64).close()
    with pytest.raises(L.LexbError):
        D.debug_fail_next(9)
    parity_still_holds(gpu, seed=4)
