"""The CPU oracle against the reference's own known-answer recipes and against two
independent restatements (numpy float16 casts; the reference test's f64 arithmetic)."""
import numpy as np
import pytest

from lex_gpu_b200 import inputs
from oracle import oracle as O


def test_e2m1_table_matches_the_literal_values():
    # crates/lex-front/src/interp.rs:30-34 ; crates/lex-front/tests/syntax.rs:509-513
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    L = O.lib()
    for c in range(16):
        got = L.lexo_e2m1(c)
        assert got == (-want[c & 7] if c & 8 else want[c & 7])
    assert np.signbit(np.float32(L.lexo_e2m1(8)))          # code 8 is -0.0


def test_e4m3_all_256_bytes():
    # crates/lex-front/src/interp.rs:37-47 ; scripts/qwen_nvfp4.py:32-40
    L = O.lib()
    for b in range(256):
        got = np.float32(L.lexo_e4m3(b))
        want = O.E4M3[b]
        if b & 0x7F == 0x7F:
            assert np.isnan(got) and np.isnan(want)
        else:
            assert got == want and np.signbit(got) == np.signbit(want), hex(b)
    assert O.E4M3[0x7E] == 448.0 and O.E4M3[0x01] == 2.0 ** -9 and O.E4M3[0x38] == 1.0


def test_f16_rounding_agrees_with_numpy_on_every_boundary():
    """Every f16 value, the midpoint to its neighbour and one f32 ulp either side of it."""
    L = O.lib()
    h = np.arange(0x0000, 0x7C00, dtype=np.uint16)
    v = h.view(np.float16).astype(np.float32)
    nxt = (h + 1).astype(np.uint16).view(np.float16).astype(np.float64)
    mid = ((v.astype(np.float64) + nxt) / 2).astype(np.float32)       # exact in f32
    cases = np.concatenate([v, mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(np.inf)),
                            np.array([65504.0, 65519.99, 65520.0, 65536.0, 1e9, 2.0 ** -25, 2.0 ** -24,
                                      np.nextafter(np.float32(2.0 ** -25), np.float32(1)), 0.0, 1e-30],
                                     dtype=np.float32)])
    cases = np.concatenate([cases, -cases])
    with np.errstate(over="ignore"):
        want = cases.astype(np.float16).view(np.uint16)
    got = np.array([L.lexo_f32_to_f16(float(c)) for c in cases], dtype=np.uint16)
    assert np.array_equal(got, want)
    back = np.array([L.lexo_f16_to_f32(int(x)) for x in h], dtype=np.float32)
    assert np.array_equal(back, v)
    assert L.lexo_f32_to_f16(float("nan")) & 0x7C00 == 0x7C00 and L.lexo_f32_to_f16(float("nan")) & 0x3FF
    assert L.lexo_f32_to_f16(float("inf")) == 0x7C00 and L.lexo_f32_to_f16(float("-inf")) == 0xFC00


def test_f16_rounding_agrees_with_numpy_on_random_f32():
    rng = np.random.Generator(np.random.PCG64(5))
    bits = rng.integers(0, 2 ** 32, size=200_000, dtype=np.uint64).astype(np.uint32)
    f = bits.view(np.float32)
    f = f[np.isfinite(f)]
    small = (rng.standard_normal(200_000) * np.exp2(rng.uniform(-26, 17, 200_000))).astype(np.float32)
    L = O.lib()
    for arr in (f[:60_000], small[:120_000]):
        with np.errstate(over="ignore"):
            want = arr.astype(np.float16).view(np.uint16)
        got = np.array([L.lexo_f32_to_f16(float(c)) for c in arr], dtype=np.uint16)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("bm,bn,bk", [(128, 128, 64), (64, 128, 32)])   # nvidia-ada, apple-m-series
def test_known_answer_recipe_of_the_reference_test(bm, bn, bk):
    """crates/lex-front/tests/syntax.rs:525-585: (m,n,k) = (bm, 2bn, 2bk); y[i,j] for i step 9,
    j step 7 within 1e-3 * max(|want|, 1) of the f64 restatement."""
    m, n, k = bm, 2 * bn, 2 * bk
    x16, q, sc, g, _ = O.kat_inputs(m, n, k)
    got = O.gemm_fp4(x16, q, sc, g, bk=bk)
    want = O.f64_restatement(x16, q, sc, g)
    sub_g, sub_w = got[::9, ::7].astype(np.float64), want[::9, ::7]
    assert np.all(np.abs(sub_g - sub_w) < 1e-3 * np.maximum(np.abs(sub_w), 1.0))
    # stronger than the reference asks: every element, and the numpy twin bit for bit
    assert np.all(np.abs(got - want) < 1e-3 * np.maximum(np.abs(want), 1.0))
    assert np.array_equal(got, O.np_gemm_fp4(x16, q, sc, g, bk=bk))
    assert np.abs(want).max() > 1e-3


@pytest.mark.parametrize("bm,bn,bk", [(128, 128, 64), (64, 128, 32)])
def test_residual_recipe_of_the_reference_test(bm, bn, bk):
    """crates/lex-front/tests/syntax.rs:634-683: with r minus with a zero r is r to 1e-5."""
    m, n, k = bm, 2 * bn, bk
    x16, q, sc, g, r = O.kat_inputs(m, n, k, residual=True)
    with_r = O.gemm_fp4(x16, q, sc, g, r=r, bk=bk)
    without = O.gemm_fp4(x16, q, sc, g, r=np.zeros_like(r), bk=bk)
    assert np.all(np.abs((with_r - without).astype(np.float64) - r) < 1e-5)
    assert np.array_equal(without, O.gemm_fp4(x16, q, sc, g, bk=bk))


def test_dequant_bits_c_vs_numpy_on_adversarial_scales():
    wq, ws, wg = inputs.adversarial_dequant_case()
    got = O.dequant_fp4_f16(wq, ws, wg)
    want = O.np_dequant_f16(wq, ws, wg).view(np.uint16)
    nan_g = (got & 0x7C00 == 0x7C00) & (got & 0x3FF != 0)
    nan_w = (want & 0x7C00 == 0x7C00) & (want & 0x3FF != 0)
    assert np.array_equal(nan_g, nan_w)
    assert np.array_equal(got[~nan_g], want[~nan_w])
    # -0 codes give f16 -0 when the scales are positive (row 0: wg = 1, scale byte 0x38 = 1.0)
    codes = O.np_codes(wq)
    col = 0x38 * 16 + int(np.where(codes[0, 0x38 * 16:0x38 * 16 + 16] == 8)[0][0])
    assert got[0, col] == 0x8000
    # the NaN scale bytes decode to NaN, not to +-480
    assert np.all(nan_g[0, 0x7F * 16:0x7F * 16 + 16]) and np.all(nan_g[0, 0xFF * 16:0xFF * 16 + 16])


def test_c_oracle_equals_numpy_twin_on_config0():
    x, wq, ws, wg = inputs.make_case(128, 128, 64)
    y = O.gemm_fp4(x, wq, ws, wg)
    assert np.array_equal(y, O.np_gemm_fp4(x, wq, ws, wg))
    assert np.abs(y).max() > 1e-3
    # thread count does not change a single bit (rows are independent)
    assert np.array_equal(y, O.gemm_fp4(x, wq, ws, wg, threads=1))


def test_row_slices_and_ragged_m():
    x, wq, ws, wg = inputs.make_case(5, 48, 128, seed_base=10)
    full = O.gemm_fp4(x, wq, ws, wg)
    part = O.gemm_fp4(x, wq, ws, wg, rows=(16, 35))
    assert np.array_equal(part[:, 16:35], full[:, 16:35]) and not part[:, :16].any() and not part[:, 35:].any()
    assert np.array_equal(full, O.np_gemm_fp4(x, wq, ws, wg))


def test_shapes_the_operator_rejects():
    x, wq, ws, wg = inputs.make_case(4, 16, 96)
    with pytest.raises(ValueError):          # k = 96 does not divide by bk = 64 (syntax.rs:1513-1516)
        O.gemm_fp4(x, wq, ws, wg, bk=64)
    with pytest.raises(ValueError):          # a rank-2 row scale is refused (tensor_shapes.rs:65-67)
        O.gemm_fp4(x, wq, ws, wg.reshape(-1, 1), bk=32)
    assert O.gemm_fp4(x, wq, ws, wg, bk=32).shape == (4, 16)


def test_metrics():
    want = np.array([1.0, -2.0, 0.0, 4.0], dtype=np.float32)
    got = np.array([1.001, -2.0, 0.0005, 4.0], dtype=np.float32)
    assert abs(O.max_rel_err(got, want) - 0.5) < 1e-6          # 0.0005 / max(0, 1e-3)
    e, scale, rel = O.err_of_scale(got, want)
    assert scale == 4.0 and abs(e - 0.001 / 4.0) < 1e-7
    assert abs(rel - 0.0005 / 4e-3) < 1e-6
    assert O.max_rel_err(np.array([np.inf], dtype=np.float32), np.array([1.0], dtype=np.float32)) == np.inf


def test_scale_generator_stays_in_the_normal_range():
    _, ws, wg = inputs.make_weights(64, 1024, seed_base=3)
    assert ws.min() >= 0x08 and ws.max() <= 0x48
    v = O.E4M3[ws]
    assert v.min() >= 2.0 ** -6 and v.max() <= 4.0
    assert wg.min() >= 0.5 and wg.max() < 2.0
    # nearest-even rounding of the generator: exact values map to themselves
    assert np.array_equal(inputs.nearest_e4m3(O.E4M3[1:0x7F].astype(np.float64)), np.arange(1, 0x7F, dtype=np.uint8))


GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def test_decode_tables_equal_the_references_python_tables():
    """tests/golden/decode_tables.npz was written by importing the reference's scripts/qwen_nvfp4.py
    (tests/golden/make_golden.py): its E2M1 and E4M3 tables, and a small matrix dequantised with them."""
    gold = np.load(GOLDEN / "decode_tables.npz")
    L = O.lib()
    assert np.array_equal(np.array([L.lexo_e2m1(c) for c in range(16)], dtype=np.float32), gold["e2m1"])
    assert np.array_equal(np.signbit(gold["e2m1"]), np.array([c >= 8 for c in range(16)]))
    ours = np.array([L.lexo_e4m3(b) for b in range(256)], dtype=np.float32)
    nan = np.isnan(gold["e4m3"])
    assert np.array_equal(np.isnan(ours), nan) and np.array_equal(ours[~nan], gold["e4m3"][~nan])
    wg = np.full(gold["wq"].shape[0], gold["gs"], dtype=np.float32)
    assert np.array_equal(O.np_dequant_f32(gold["wq"], gold["ws"], wg), gold["w_f32"])
    with np.errstate(over="ignore"):
        assert np.array_equal(O.dequant_fp4_f16(gold["wq"], gold["ws"], wg), gold["w_f32"].astype(np.float16).view(np.uint16))


def test_config0_regression_pin():
    gold = np.load(GOLDEN / "config0.npz")
    x, wq, ws, wg = inputs.make_case(128, 128, 64)
    assert np.array_equal(O.gemm_fp4(x, wq, ws, wg), gold["y"])
    assert np.array_equal(O.dequant_fp4_f16(wq, ws, wg), gold["w16"])


# ---------------------------------------------------------------- matmul_q_x (NVFP4 layout)

def test_matmul_q_x_matches_f64_and_keeps_f32_weights():
    from lex_gpu_b200 import inputs
    x, wq, ws, wg = inputs.make_case(3, 64, 1024, seed_base=900)
    y = O.matmul_q_x(x, wq, ws, wg)
    w = O.np_dequant_f32(wq, ws, wg).astype(np.float64)
    ref = x.astype(np.float64) @ w.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 2e-6       # only the f32 sums round
    # gemm_fp4 rounds the weights to f16 on top of that: visibly further from exact arithmetic
    y16 = O.gemm_fp4(x, wq, ws, wg)
    assert np.abs(y16 - ref).max() / np.abs(ref).max() > 2e-5
    assert O.err_of_scale(y16, y)[0] < 2e-3                        # and still inside the reference gate


def test_matmul_q_x_chunks_residual_and_f32_x():
    from lex_gpu_b200 import inputs
    x, wq, ws, wg = inputs.make_case(2, 32, 512, seed_base=901)
    r = np.arange(64, dtype=np.float32).reshape(2, 32)
    whole = O.matmul_q_x(x, wq, ws, wg, r=r)
    chunked = O.matmul_q_x(x, wq, ws, wg, r=r, kc=128)             # same value up to the order of the f32 sums
    assert np.abs(whole - chunked).max() / np.abs(whole).max() < 1e-5
    assert np.array_equal(O.matmul_q_x(x.astype(np.float32), wq, ws, wg, r=r), whole)   # widening f16 is exact
    # the sequential sum of one chunk, restated in numpy
    w = O.np_dequant_f32(wq, ws, wg)
    acc = np.float32(0)
    for p in range(512):
        acc = np.float32(acc + np.float32(np.float32(x[1, p]) * w[7, p]))
    assert np.float32(acc + r[1, 7]) == whole[1, 7]
    with pytest.raises(ValueError):
        O.matmul_q_x(x, wq, ws, wg, kc=100)                        # must divide k in groups of 16 (llama.rs:407-413)


def test_matmul_q_x_on_the_reference_gpu_test_recipes():
    """crates/lex-cuda/tests/device_gpu.rs:131-209: the recipes feed scale bytes with the sign bit set."""
    x = O.ref_fill(512, 5).reshape(1, 512)
    assert x.min() >= -1 and x.max() < 1 and x[0, 0] == np.float32(5 >> 9) / np.float32(4194304.0) - 1
    wq, ws = O.ref_nvfp4_bytes(64, 512, 31, 7, 0x38, 5)
    assert wq[0, 0] == ((7 - 128) & 0xFF) and set(np.unique(ws)) == {0xB8, 0xB9, 0xBA, 0xBB, 0xBC}
    wg = np.ones(64, dtype=np.float32)
    y = O.matmul_q_x(x, wq, ws, wg)
    w = O.np_dequant_f32(wq, ws, wg).astype(np.float64)
    assert w[0, 0] == -6.0 and w[0, 1] == 0.0                        # code 7 (6.0), then code 8 (-0), times the scale byte 0xb8 = -1
    ref = x.astype(np.float64) @ w.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-6
    assert np.abs(ref).max() > 1.0


def test_quant16_restatement_properties():
    """crates/lex-msl/src/int8.rs:47-114: int16 codes within +-32767, the group's largest value on the end of the
    range, a group of zeros gives scale 0 and codes 0, and xq * xs is within half a step of x."""
    rng = np.random.Generator(np.random.PCG64(9))
    x = (rng.standard_normal((4, 256)) * np.exp2(rng.integers(-10, 6, (4, 256)))).astype(np.float32)
    x[0, :16] = 0
    xq, xs = O.np_quant16(x)
    assert xq.dtype == np.int16 and xs.dtype == np.float32 and xs.shape == (4, 16)
    assert np.abs(xq.astype(np.int32)).max() == 32767 and not xq[0, :16].any() and xs[0, 0] == 0
    back = xq.astype(np.float64) * np.repeat(xs.astype(np.float64), 16, axis=1)
    assert np.all(np.abs(back - x) <= 0.5000001 * np.repeat(xs, 16, axis=1) + 1e-30)
    assert np.array_equal(np.abs(xq).reshape(4, 16, 16).max(axis=2)[xs > 0], np.full((xs > 0).sum(), 32767))
    with pytest.raises(ValueError):
        O.np_quant16(np.zeros((1, 48), dtype=np.float32))
