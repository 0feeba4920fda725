"""The integer-activation path of the reference (lex_msl::int8, crates/lex-msl/src/int8.rs): quant16 and
matmul_int8, through the C ABI.

quant16 is held to a numpy restatement bit for bit (its outputs are an interface: xq and xs are bound to the
matmul).  matmul_int8 is held to the reference's own test for it
(`the_int8_matmul_matches_the_matmul_and_ignores_its_batch`, crates/lex-cuda/tests/device_gpu.rs:314-420): same
input recipes, the interpreter's matmul_q_x on the unquantised activations as the expected value, 2e-3 of scale,
and a token's output bit-identical alone and in a batch - plus a tighter comparison with the int16 arithmetic
itself in f64.
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


def quant_on_device(gpu, x):
    m, k = x.shape
    xb = gpu.upload(x)
    xq, xs = gpu.alloc(m * k * 2), gpu.alloc(m * (k // 16) * 4)
    gpu.quant16(m, k, xb, xq, xs, x_half=x.dtype == np.float16)
    return xq, xs


def int8_matmul(gpu, x, wq, ws, wg, r=None, **sched):
    m, k = x.shape
    n = wq.shape[0]
    xq, xs = quant_on_device(gpu, x)
    q = L.QBuf(gpu, wq, ws, wg)
    yb = gpu.alloc(4 * m * n)
    gpu.memset(yb, 0xEE)
    pipe = gpu.plan_matmul_int8(m, n, k, r is not None, **sched)
    bufs = [xq, xs, q.wq, q.ws, q.wg] + ([gpu.upload(np.ascontiguousarray(r, dtype=np.float32))] if r is not None else []) + [yb]
    gpu.run_launches([(pipe, bufs)])
    y = gpu.download(yb, np.float32, (m, n))
    assert gpu.status_word() == 0
    return y, gpu.download(xq, np.int16, (m, k)), gpu.download(xs, np.float32, (m, k // 16))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_quant16_bit_for_bit(gpu, dtype):
    rng = np.random.Generator(np.random.PCG64(600))
    x = (rng.standard_normal((5, 2048)) * np.exp2(rng.integers(-12, 8, (5, 2048)))).astype(dtype)
    x[0, :16] = 0                                     # a group of zeros: scale 0, codes 0
    x[1, 16:32] = dtype(3.0)                          # every value the group's maximum
    x[2, 32:48] = np.linspace(-1, 1, 16).astype(dtype)
    x[3, 48:64] = (np.arange(16) - 7.5).astype(dtype)  # ties at the half steps
    xq, xs = quant_on_device(gpu, x)
    got_q, got_s = gpu.download(xq, np.int16, x.shape), gpu.download(xs, np.float32, (5, 2048 // 16))
    want_q, want_s = O.np_quant16(x)
    assert np.array_equal(got_s, want_s)
    assert np.array_equal(got_q, want_q)
    assert np.abs(got_q.astype(np.int32)).max() == 32767 and not got_q[0, :16].any() and got_s[0, 0] == 0
    with pytest.raises(L.LexbError):
        gpu.quant16(1, 48, xq, xq, xs, x_half=False)


def test_the_int8_matmul_matches_the_matmul_and_ignores_its_batch(gpu):
    """The reference's own test (device_gpu.rs:314-420) with 128 output rows for its 96."""
    n, k = 128, 1024
    wq, ws = O.ref_nvfp4_bytes(n, k, 97, 3, 0x34, 7)
    wg = (0.5 + (np.arange(n) % 5).astype(np.float32) * np.float32(0.125)).astype(np.float32)
    alone = None
    for m, residual, x_half in [(1, False, False), (3, False, True), (3, True, False), (8, True, True), (3, False, False)]:
        x = O.ref_fill(m * k, 3).reshape(m, k)
        r = O.ref_fill(m * n, 11).reshape(m, n) if residual else None
        xin = x.astype(np.float16) if x_half else x
        got, _, _ = int8_matmul(gpu, xin, wq, ws, wg, r)
        want = O.matmul_q_x(xin, wq, ws, wg, r=r)
        err, scale, _ = O.err_of_scale(got, want)
        print(f"  int8 m={m} residual={residual} x_half={x_half}: {err:.3e} of scale")
        assert scale > 1e-3 and err < 2e-3
        if not residual and not x_half:
            if alone is None:
                alone = got[0].copy()
            else:
                assert np.array_equal(alone, got[0]), "a token's output depends on its batch"
    assert alone is not None


@pytest.mark.parametrize("m,n,k,residual", [(1, 256, 2048, False), (4, 384, 1024, True), (8, 128, 5120, False), (16, 256, 1024, False)])
def test_int8_matmul_against_the_int16_arithmetic_itself(gpu, m, n, k, residual):
    """Against the f64 value of sum (xq * xs) * w: the digit rows keep 16 bits below each group's largest
    value, so the result lies within 1e-4 of scale of the int16 arithmetic (the reference's bar is 2e-3)."""
    x = inputs.make_x(m, k, seed_base=610 + m).astype(np.float32)
    wq, ws, wg = inputs.make_weights(n, k, seed_base=611)
    r = inputs.make_residual(m, n, seed_base=612) if residual else None
    got, xq, xs = int8_matmul(gpu, x, wq, ws, wg, r)
    want = O.np_matmul_int8_f64(xq, xs, wq, ws, wg, r)
    scale = np.abs(want).max()
    err = np.abs(got - want).max() / scale
    print(f"  against the int16 arithmetic in f64: {err:.3e} of scale")
    assert scale > 1e-3 and err <= 1e-4
    e2, s2, _ = O.err_of_scale(got, O.matmul_q_x(x, wq, ws, wg, r=r))
    assert e2 < 2e-3


@pytest.mark.parametrize("m", [1, 4])
def test_int8_matmul_decode_shape(gpu, m):
    """The decode / verify shape of the 27B MLP (n = 17408, k = 5120) at full size."""
    n, k = 17408, 5120
    x = inputs.make_x(m, k, seed_base=620).astype(np.float32)
    wq, ws, wg = inputs.make_weights(n, k)
    got, xq, xs = int8_matmul(gpu, x, wq, ws, wg)
    err, scale, _ = O.err_of_scale(got, O.matmul_q_x(x, wq, ws, wg))
    print(f"  m={m}: {err:.3e} of scale against the interpreter's matmul_q_x")
    assert scale > 1e-3 and err < 2e-3


def test_int8_pipeline_describes_itself_and_checks_its_bindings(gpu):
    pipe = gpu.plan_matmul_int8(3, 256, 1024, residual=True)
    d = pipe.describe()
    assert d.entry.decode() == "matmul_int8_3x256x1024_res" and d.nbind == 7 and list(d.writes)[:7] == [0, 0, 0, 0, 0, 0, 1]
    b = gpu.alloc(1 << 20)
    with pytest.raises(L.LexbError) as e:
        gpu.run_launches([(pipe, [b, b, b, b, b, b])])          # six buffers where seven are bound
    assert e.value.code == 1 and "xq, xs" in e.value.message
    with pytest.raises(L.LexbError):
        gpu.plan_matmul_int8(3, 100, 1024)                       # n % 128
    assert gpu.status_word() == 0
