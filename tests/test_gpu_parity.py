"""Parity of the CUDA kernels with the CPU oracle, through the C ABI.

Gates (the reference's GEMM convention, crates/lex-cuda/tests/device_gpu.rs:294-303):
  * of scale:  max|got - want| / max|want| <= 2e-3, after asserting max|want| > 1e-3;
  * per element with a floor tied to the output scale: |d| / max(|want|, 1e-3 max|want|) <= 2e-3
    for k < 4096.  The tensor core adds into its f32 accumulator without rounding to
    nearest, so the error of one accumulator grows with the number of K steps it sees; for
    long contractions (k >= 4096) this metric is gated at 1e-2 (LONG_K_REL) and the measured
    value is printed;
  * dequantised weights: every f16 bit pattern equal (-0 != +0; NaN matches NaN).
"""
import numpy as np
import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import inputs
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3
LONG_K_REL = 1e-2


@pytest.fixture(scope="module")
def gpu():
    from lex_gpu_b200 import build
    build.build()
    g = L.Gpu(0)
    yield g
    g.close()


def check(got, want, tol=TOL, rel_tol=TOL):
    assert np.isfinite(got).all(), "non-finite output (an element was not written?)"
    err, scale, rel = O.err_of_scale(got, want)
    print(f"  {err:.3e} of scale, {rel:.3e} per element (floor 1e-3 of scale), raw max_rel_err {O.max_rel_err(got, want):.3e}")
    assert scale > 1e-3, "the reference output is all but zero"
    assert err <= tol, f"{err:e} of scale"
    assert rel <= rel_tol, f"per-element relative error {rel:e}"
    return err


def same_f16_bits(got, want):
    nan_g = (got & 0x7C00 == 0x7C00) & (got & 0x3FF != 0)
    nan_w = (want & 0x7C00 == 0x7C00) & (want & 0x3FF != 0)
    return np.array_equal(nan_g, nan_w) and np.array_equal(got[~nan_g], want[~nan_w])


# ---------------------------------------------------------------- dequant: bit-exact

def test_dequant_bit_exact_adversarial(gpu):
    wq, ws, wg = inputs.adversarial_dequant_case()
    got = L.dequant_fp4_f16(gpu, wq, ws, wg)
    want = O.dequant_fp4_f16(wq, ws, wg)
    assert same_f16_bits(got, want)
    assert (want == 0x8000).any() and (want == 0x0000).any()      # both zeros occur


def test_dequant_bit_exact_benchmark_distribution(gpu):
    wq, ws, wg = inputs.make_weights(2048, 5120, seed_base=0)
    got = L.dequant_fp4_f16(gpu, wq, ws, wg)
    assert np.array_equal(got, O.dequant_fp4_f16(wq, ws, wg))


def test_dequant_rejects_k_not_multiple_of_16(gpu):
    with pytest.raises(L.LexbError):
        b = gpu.alloc(1024)
        gpu.dequant_fp4_f16(4, 24, b, b, b, b)


# ---------------------------------------------------------------- matvec path (m <= 16)

@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 9, 16])
def test_matvec_small_shapes(gpu, m):
    x, wq, ws, wg = inputs.make_case(m, 256, 1024, seed_base=20 + m)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    check(got, O.gemm_fp4(x, wq, ws, wg))


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (4, 48, 64), (2, 32, 96), (5, 64, 160), (16, 16, 2080), (3, 128, 3072)])
def test_matvec_ragged_k(gpu, m, n, k):
    """k a multiple of 32 only: slices that end inside a warp's 128 columns; bk = 32 in the oracle."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=31)
    check(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg, bk=32))


@pytest.mark.parametrize("m,kc", [(4, 1024), (16, 1024), (16, 2048), (1, 4096)])
def test_matvec_chunked_x(gpu, m, kc):
    x, wq, ws, wg = inputs.make_case(m, 64, 5120, seed_base=41)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kc=kc), O.gemm_fp4(x, wq, ws, wg))


def test_matvec_residual(gpu):
    x, wq, ws, wg = inputs.make_case(4, 128, 512, seed_base=51)
    r = inputs.make_residual(4, 128, seed_base=51)
    got = L.gemm_fp4(gpu, x, wq, ws, wg, r=r)
    want = O.gemm_fp4(x, wq, ws, wg, r=r)
    check(got, want)
    base = L.gemm_fp4(gpu, x, wq, ws, wg)
    assert np.allclose(got - base, r, atol=1e-4)


@pytest.mark.parametrize("m", [1, 4])
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
def test_matvec_benchmark_shapes(gpu, m, n, k):
    """The decode / spec-verify matvec configuration (m in {1, 4} at the 27B MLP shapes) at full size, against the full oracle."""
    x, wq, ws, wg = inputs.make_case(m, n, k)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    check(got, O.gemm_fp4(x, wq, ws, wg))


def test_a_token_does_not_depend_on_its_batch(gpu):
    """The int8 test idea of crates/lex-cuda/tests/device_gpu.rs:314-: a row's result is the same
    whatever else is in the batch - bit for bit within the matvec path."""
    x, wq, ws, wg = inputs.make_case(8, 256, 2048, seed_base=61)
    y8 = L.gemm_fp4(gpu, x, wq, ws, wg)
    y1 = L.gemm_fp4(gpu, x[:1].copy(), wq, ws, wg)
    y4 = L.gemm_fp4(gpu, x[:4].copy(), wq, ws, wg)
    assert np.array_equal(y1, y8[:1]) and np.array_equal(y4, y8[:4])


# ---------------------------------------------------------------- tcgen05 path (m > 16)

def test_gemm_config0_readme_example(gpu):
    """m = n = 128, k = 64: one tile, one K step (the README's CPU-interpreter example); also against the committed fixture."""
    from pathlib import Path
    x, wq, ws, wg = inputs.make_case(128, 128, 64)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    check(got, O.gemm_fp4(x, wq, ws, wg))
    gold = np.load(Path(__file__).resolve().parent / "golden" / "config0.npz")
    check(got, gold["y"])
    assert np.array_equal(L.dequant_fp4_f16(gpu, wq, ws, wg), gold["w16"])


@pytest.mark.parametrize("bm,bn,bk", [(128, 128, 64)])
def test_gemm_known_answer_recipe(gpu, bm, bn, bk):
    """Inputs of crates/lex-front/tests/syntax.rs:525-585 with its own tolerance against the f64 restatement."""
    m, n, k = bm, 2 * bn, 2 * bk
    x16, q, sc, g, _ = O.kat_inputs(m, n, k)
    got = L.gemm_fp4(gpu, x16, q, sc, g)
    want = O.f64_restatement(x16, q, sc, g)
    assert np.all(np.abs(got - want) < 1e-3 * np.maximum(np.abs(want), 1.0))
    check(got, O.gemm_fp4(x16, q, sc, g))


def test_gemm_residual_recipe(gpu):
    """crates/lex-front/tests/syntax.rs:634-683: the residual is added exactly once."""
    m, n, k = 128, 256, 64
    x16, q, sc, g, r = O.kat_inputs(m, n, k, residual=True)
    with_r = L.gemm_fp4(gpu, x16, q, sc, g, r=r)
    without = L.gemm_fp4(gpu, x16, q, sc, g, r=np.zeros_like(r))
    assert np.all(np.abs((with_r - without).astype(np.float64) - r) < 1e-5)
    check(with_r, O.gemm_fp4(x16, q, sc, g, r=r))


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (17, 128, 256), (40, 128, 512), (96, 256, 1024),
                                   (300, 384, 2048), (512, 1024, 5120), (1000, 256, 320)])
def test_gemm_shapes(gpu, m, n, k):
    """Multi-tile, multi-K-step and ragged m (the reference's ragged cases,
    crates/lex-cuda/tests/device_gpu.rs:210-305, restricted to n % 128 == 0, k % 64 == 0)."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=m + n)
    check(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg), rel_tol=TOL if k < 4096 else LONG_K_REL)


@pytest.mark.parametrize("m,n,k", [(512, 256, 256), (512, 256, 512), (300, 256, 1024), (257, 512, 768),
                                   (1000, 512, 2048), (1024, 768, 1280), (128, 256, 256)])
def test_gemm_two_cta_kernel(gpu, m, n, k):
    """The cta_group::2 kernel (pairs of CTAs, 512 tokens per tile), forced; partial token tiles,
    several pairs, several m tiles; the one-CTA kernel must agree with it to tolerance too."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=m + k)
    want = O.gemm_fp4(x, wq, ws, wg)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=3), want)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=2), want)


@pytest.mark.parametrize("m,n,k,tm,splits", [(64, 256, 512, 64, 0), (128, 256, 1024, 128, 0), (100, 384, 768, 64, 0),
                                             (100, 384, 768, 128, 0), (512, 512, 2048, 128, 2), (512, 256, 1024, 64, 0),
                                             (300, 256, 1024, 128, 3), (17, 256, 512, 0, 0), (48, 128, 256, 0, 0),
                                             (129, 256, 768, 0, 0)])
def test_gemm_two_cta_kernel_tiles_of_128_and_64_tokens(gpu, m, n, k, tm, splits):
    """The narrower tiles (MMAs of N = 128 / 64, x boxes of 64 / 32 tokens per CTA), forced and as the planner picks them
    for small m: partial last tiles, several tiles of tokens, split K, residual."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=m + k + tm)
    r = inputs.make_residual(m, n, seed_base=3)
    d = gpu.plan_gemm_fp4(m, n, k, kernel=3, tm=tm, k_splits=splits).describe()
    assert int(d.entry.decode().split("_")[-3]) in ((tm,) if tm else (64, 128, 256))
    check(L.gemm_fp4(gpu, x, wq, ws, wg, r=r, kernel=3, tm=tm, k_splits=splits), O.gemm_fp4(x, wq, ws, wg, r=r))
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=3, tm=tm, k_splits=splits), O.gemm_fp4(x, wq, ws, wg))


def test_gemm_two_cta_kernel_seeded_random_plans(gpu):
    """Forty seeded draws of (m, n, k, tile, K split, ring depths, residual) for the two-CTA kernel against the oracle:
    every tile size with every stage layout it can take, odd last pairs, partial token tiles."""
    rng = np.random.Generator(np.random.PCG64(20240611))
    done = 0
    for draw in range(200):
        if done == 40:
            break
        m = int(rng.integers(9, 700))
        n = 128 * int(rng.integers(1, 9))
        k = 256 * int(rng.integers(1, 13))
        tm = int(rng.choice([0, 64, 128, 256, 512]))
        splits = int(rng.choice([0, 0, 1, 2, 3]))
        stages, w_stages = (int(rng.integers(2, 7)), int(rng.integers(2, 9))) if rng.random() < 0.5 else (0, 0)
        with_r = bool(rng.random() < 0.5)
        try:
            gpu.plan_gemm_fp4(m, n, k, with_r, kernel=3, tm=tm, k_splits=splits, stages=stages, w_stages=w_stages)
        except L.LexbError:
            continue                                  # a combination the planner refuses (shared memory, splits > blocks)
        x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=1000 + draw)
        r = inputs.make_residual(m, n, seed_base=draw) if with_r else None
        got = L.gemm_fp4(gpu, x, wq, ws, wg, r=r, kernel=3, tm=tm, k_splits=splits, stages=stages, w_stages=w_stages)
        print(f"  draw {draw}: m={m} n={n} k={k} tm={tm} splits={splits} stages={stages}/{w_stages} r={with_r}")
        check(got, O.gemm_fp4(x, wq, ws, wg, r=r), rel_tol=TOL if k < 2048 else LONG_K_REL)
        done += 1
    assert done == 40


@pytest.mark.parametrize("tm", [256, 512])
def test_gemm_two_cta_kernel_residual_and_stages(gpu, tm):
    """Ring depths around the defaults, for both tile sizes: (2, 2) makes the barrier rings (at least 4 deep) deeper
    than both data rings, (3, 5) and (6, 5) make the W ring deeper than the four decode groups, (4, 2) has fewer W
    stages than groups.  28 K steps: every ring wraps several times."""
    m, n, k = 640, 512, 1792
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=77)
    r = inputs.make_residual(m, n, seed_base=77)
    want = O.gemm_fp4(x, wq, ws, wg, r=r)
    for stages, w_stages in ((2, 2), (3, 5), (4, 2), (2, 6), (6, 5) if tm == 256 else (3, 4), (0, 0)):
        check(L.gemm_fp4(gpu, x, wq, ws, wg, r=r, kernel=3, tm=tm, stages=stages, w_stages=w_stages), want)


@pytest.mark.parametrize("m,n,k,splits", [(512, 256, 2048, 2), (600, 384, 4096, 4), (512, 384, 512, 1),
                                          (300, 128, 1024, 3), (512, 640, 2304, 5)])
def test_gemm_two_cta_split_k_and_odd_last_pair(gpu, m, n, k, splits):
    """K split across CTA pairs (partials in the pipeline's workspace, summed by a second launch),
    n an odd number of 128-row tiles (the last pair has one idle half), with and without r."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=n + k)
    r = inputs.make_residual(m, n, seed_base=5)
    rel = TOL if k < 4096 else LONG_K_REL
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=3, k_splits=splits), O.gemm_fp4(x, wq, ws, wg), rel_tol=rel)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, r=r, kernel=3, k_splits=splits), O.gemm_fp4(x, wq, ws, wg, r=r), rel_tol=rel)


def test_split_k_is_chosen_for_few_tiles(gpu):
    d = gpu.plan_gemm_fp4(512, 5120, 17408).describe()          # 20 pairs on 74 SM pairs
    assert d.kernel == 3 and d.k_splits == 3 and d.scratch_bytes == 3 * 512 * 5120 * 4 and d.grid == 120
    d = gpu.plan_gemm_fp4(512, 17408, 5120).describe()
    assert d.k_splits == 1 and d.scratch_bytes == 0


def test_two_cta_kernel_multiplies_exactly_the_oracles_f16_weights(gpu):
    n, k = 512, 512
    wq, ws, wg = inputs.make_weights(n, k, seed_base=92)
    x = np.zeros((k, k), dtype=np.float16)
    x[np.arange(k), np.arange(k)] = 1.0
    got = L.gemm_fp4(gpu, x, wq, ws, wg, kernel=3)
    want = O.dequant_fp4_f16(wq, ws, wg).view(np.float16).astype(np.float32).T
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tm,stages", [(16, 2), (32, 3), (64, 0), (128, 4), (256, 2), (256, 0), (112, 0)])
def test_gemm_schedules(gpu, tm, stages):
    x, wq, ws, wg = inputs.make_case(200, 256, 1536, seed_base=71)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=2, tm=tm, stages=stages), O.gemm_fp4(x, wq, ws, wg))


def test_gemm_small_m_through_the_tensor_path(gpu):
    """m <= 16 forced onto the tcgen05 kernel agrees with the matvec kernel to tolerance."""
    x, wq, ws, wg = inputs.make_case(16, 256, 1024, seed_base=81)
    want = O.gemm_fp4(x, wq, ws, wg)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=2), want)
    check(L.gemm_fp4(gpu, x, wq, ws, wg, kernel=1), want)


def test_gemm_multiplies_exactly_the_oracles_f16_weights(gpu):
    """x = one-hot rows: y[i, j] is then the staged weight W[j, k_i] itself, so the tensor-core
    path reproduces the oracle's f16 weights exactly (only the sign of zero is lost in a sum)."""
    n, k = 256, 512
    wq, ws, wg = inputs.make_weights(n, k, seed_base=91)
    x = np.zeros((k, k), dtype=np.float16)
    x[np.arange(k), np.arange(k)] = 1.0
    got = L.gemm_fp4(gpu, x, wq, ws, wg)                        # [k, n] = W^T
    want = O.dequant_fp4_f16(wq, ws, wg).view(np.float16).astype(np.float32).T
    assert np.array_equal(got, want)


def test_gemm_wide_scale_range(gpu):
    """Every finite scale byte (E4M3 subnormals and negative scales included) and row scales of
    both signs over three decades, through the MMA path: f16-subnormal and large weights mix."""
    n, k, m = 256, 2048, 64
    rng = np.random.Generator(np.random.PCG64(95))
    finite = np.array([b for b in range(256) if b & 0x7F != 0x7F], dtype=np.uint8)
    ws = rng.choice(finite, size=(n, k // 16))
    wq = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    wg = (np.exp(rng.uniform(np.log(1e-3), 0.0, n)) * rng.choice([-1.0, 1.0], n)).astype(np.float32)
    x = inputs.make_x(m, k, seed_base=95)
    assert np.array_equal(L.dequant_fp4_f16(gpu, wq, ws, wg), O.dequant_fp4_f16(wq, ws, wg))
    check(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg))
    check(L.gemm_fp4(gpu, x[:8].copy(), wq, ws, wg), O.gemm_fp4(x[:8].copy(), wq, ws, wg))


@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
def test_gemm_27b_mlp_prefill_m512(gpu, n, k):
    """The 27B MLP prefill configuration (m = 512) at full size against the full oracle."""
    x, wq, ws, wg = inputs.make_case(512, n, k)
    check(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg), rel_tol=LONG_K_REL)


@pytest.mark.parametrize("n,k", [(6144, 4096), (28672, 4096), (4096, 14336)])
def test_gemm_llama8b_prefill_projections(gpu, n, k):
    """The Llama-3.1-8B-shaped prefill projections at m = 512: oracle on a slice of rows (full n on the GPU)."""
    x, wq, ws, wg = inputs.make_case(512, n, k, seed_base=2)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    lo, hi = n // 2 - 256, n // 2 + 256
    want = O.gemm_fp4(x, wq, ws, wg, rows=(lo, hi))
    rel = LONG_K_REL
    check(got[:, lo:hi], want[:, lo:hi], rel_tol=rel)
    first = O.gemm_fp4(x, wq, ws, wg, rows=(0, 128))
    check(got[:, :128], first[:, :128], rel_tol=rel)
    last = O.gemm_fp4(x, wq, ws, wg, rows=(n - 128, n))
    check(got[:, n - 128:], last[:, n - 128:], rel_tol=rel)


def test_gemm_m2048_linearity_and_slices(gpu):
    """m = 2048 (the larger prefill batch): oracle on row slices, and the size-independent
    property that the result for a sub-batch equals the same rows of the full batch."""
    n, k = 5120, 17408
    x, wq, ws, wg = inputs.make_case(2048, n, k, seed_base=3)
    got = L.gemm_fp4(gpu, x, wq, ws, wg, k_splits=1)
    want = O.gemm_fp4(x, wq, ws, wg, rows=(1024, 1280))
    check(got[:, 1024:1280], want[:, 1024:1280], rel_tol=LONG_K_REL)
    sub = L.gemm_fp4(gpu, x[512:1024].copy(), wq, ws, wg, k_splits=1)      # same K order as the full batch
    assert np.array_equal(sub, got[512:1024])


# ---------------------------------------------------------------- boundary behaviour

def test_shapes_the_operator_rejects(gpu):
    for m, n, k in [(64, 100, 128), (64, 128, 96), (4, 40, 64), (4, 32, 48), (0, 128, 64)]:
        with pytest.raises(L.LexbError) as e:
            gpu.plan_gemm_fp4(m, n, k)
        assert e.value.code == 2, (m, n, k)
    with pytest.raises(L.LexbError):
        gpu.plan_gemm_fp4(64, 128, 64, kernel=1)        # matvec kernel takes m <= 16
    with pytest.raises(L.LexbError):
        gpu.plan_gemm_fp4(64, 128, 64, tm=24)
    with pytest.raises(L.LexbError):
        gpu.plan_gemm_fp4(512, 256, 320, kernel=3)      # the two-CTA kernel takes k in blocks of 256


def test_launch_validates_bindings(gpu):
    pipe = gpu.plan_gemm_fp4(32, 128, 64)
    small = gpu.alloc(64)
    ok = gpu.alloc(32 * 128 * 4)
    with pytest.raises(L.LexbError) as e:
        gpu.run(pipe, [small, ok, ok, ok, ok])
    assert "x" in e.value.message and e.value.code == 1
    with pytest.raises(L.LexbError):
        gpu.run(pipe, [ok, ok, ok, ok, ok, ok])          # a residual bound to a pipeline without one
    with pytest.raises(L.LexbError):
        gpu.run(pipe, [ok, ok, ok])


def test_describe_mirrors_the_lowered_descriptor(gpu):
    d = gpu.plan_gemm_fp4(512, 17408, 5120).describe()
    assert d.entry.decode() == "gemm_fp4_512_17408_5120_512_256_64"
    assert (d.grid, d.grid2, d.threads, d.nbind) == (136, 1, 608, 5)
    assert list(d.writes)[:5] == [0, 0, 0, 0, 1] and d.kernel == 3
    d = gpu.plan_gemm_fp4(256, 17408, 5120).describe()
    assert d.entry.decode() == "gemm_fp4_256_17408_5120_256_256_64" and d.kernel == 3 and d.grid == 136
    d = gpu.plan_gemm_fp4(64, 17408, 5120).describe()
    assert d.entry.decode() == "gemm_fp4_64_17408_5120_64_256_64" and d.kernel == 3 and d.grid == 136      # 64-token tiles
    d = gpu.plan_gemm_fp4(128, 17408, 5120).describe()
    assert d.entry.decode() == "gemm_fp4_128_17408_5120_128_256_64" and d.grid == 136
    assert gpu.plan_gemm_fp4(64, 2176, 5120).describe().kernel == 3         # few tiles: split K on CTA pairs
    assert gpu.plan_gemm_fp4(64, 256, 320).describe().kernel == 2           # k not in blocks of 256
    d = gpu.plan_gemm_fp4(4, 17408, 5120, residual=True).describe()
    assert d.entry.decode().startswith("gemm_fp4_res_4_17408_5120") and d.kernel == 1
    assert d.nbind == 6 and list(d.writes)[:6] == [0, 0, 0, 0, 0, 1] and 0 < d.grid <= 1088 and 1088 % d.grid in range(d.grid)


def test_run_launches_and_timing_entry_points(gpu):
    x, wq, ws, wg = inputs.make_case(64, 256, 512, seed_base=7)
    q = L.QBuf(gpu, wq, ws, wg)
    xb, yb = gpu.upload(x), gpu.zeroed(64 * 256 * 4)
    pipe = gpu.plan_gemm_fp4(64, 256, 512)
    steps = [(pipe, q.bind(xb, None, yb))] * 3
    cpu_s, wall_s = gpu.run_launches(steps)
    assert 0 <= cpu_s <= wall_s
    each = gpu.run_each_timed(steps)
    assert len(each) == 3 and all(t > 0 for t in each)
    assert gpu.time_launches(steps, reps=2) > 0
    check(gpu.download(yb, np.float32, (64, 256)), O.gemm_fp4(x, wq, ws, wg))
    assert gpu.status_word() == 0


def test_run_host_copies_in_and_out(gpu):
    m, n, k = 64, 256, 512
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=8)
    q = L.QBuf(gpu, wq, ws, wg)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    hx, hy = L.HostBuffer(x.nbytes), L.HostBuffer(m * n * 4)
    hx.array(np.float16, (m, k))[:] = x
    xd, yd = gpu.alloc(x.nbytes), gpu.alloc(m * n * 4)
    gpu.run_host(pipe, hx.ptr, xd, q.wq, q.ws, q.wg, None, yd, hy.ptr)
    check(hy.array(np.float32, (m, n)).copy(), O.gemm_fp4(x, wq, ws, wg))


def test_torch_default_stream_is_passed_as_the_legacy_stream(gpu):
    """torch's default stream has the handle 0, which means "the library's own stream" to lexb_set_stream: the
    binding passes cudaStreamLegacy instead, so that launches are ordered with torch's work on that stream.
    A torch fill, the launch and a torch read follow one another with no synchronise in between."""
    import torch
    m, n, k = 64, 512, 1024
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=14)
    q = L.QBuf(gpu, wq, ws, wg)
    xb = gpu.upload(x)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    assert torch.cuda.current_stream().cuda_stream == 0
    gpu.set_stream(torch.cuda.current_stream().cuda_stream)
    try:
        assert gpu._L.lexb_get_stream(gpu.handle) == 1
        y = torch.empty((m, n), dtype=torch.float32, device="cuda")
        for _ in range(3):
            y.fill_(float("nan"))
            gpu.run(pipe, q.bind(xb, None, gpu.wrap_tensor(y)))
            got = y.clone()                    # torch's copy on the default stream, ordered after the launch
            torch.cuda.synchronize()
            check(got.cpu().numpy(), O.gemm_fp4(x, wq, ws, wg))
    finally:
        gpu.set_stream(None)


def test_enqueue_host_on_two_streams(gpu):
    """Double-buffered chunks: two streams, two sets of staging buffers, no wait between the chunks."""
    import torch
    m, n, k = 96, 512, 1024
    wq, ws, wg = inputs.make_weights(n, k, seed_base=12)
    q = L.QBuf(gpu, wq, ws, wg)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    xs = [inputs.make_x(m, k, seed_base=20 + i) for i in range(5)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    lanes = [(L.HostBuffer(m * k * 2), L.HostBuffer(m * n * 4), gpu.alloc(m * k * 2), gpu.alloc(m * n * 4)) for _ in range(2)]
    got = []
    try:
        for i, x in enumerate(xs):
            hx, hy, xd, yd = lanes[i % 2]
            if i >= 2:                                  # the lane's previous chunk must be out before its buffers are reused
                streams[i % 2].synchronize()
                got.append(hy.array(np.float32, (m, n)).copy())
            hx.array(np.float16, (m, k))[:] = x
            gpu.set_stream(streams[i % 2].cuda_stream)
            gpu.enqueue_host(pipe, hx.ptr, xd, q.wq, q.ws, q.wg, None, yd, hy.ptr)
        for i in range(len(xs) - 2, len(xs)):
            streams[i % 2].synchronize()
            got.append(lanes[i % 2][1].array(np.float32, (m, n)).copy())
    finally:
        gpu.set_stream(None)
    for x, y in zip(xs, got):
        check(y, O.gemm_fp4(x, wq, ws, wg))
    assert gpu.status_word() == 0


def test_wrapping_a_torch_tensor(gpu):
    import torch
    m, n, k = 32, 128, 256
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=9)
    dev = torch.device("cuda:0")
    tx = torch.from_numpy(x.view(np.int16)).to(dev)
    tq, ts, tg = (torch.from_numpy(a).to(dev) for a in (wq, ws, wg))
    ty = torch.full((m, n), float("nan"), device=dev)
    torch.cuda.synchronize()
    pipe = gpu.plan_gemm_fp4(m, n, k)
    gpu.run(pipe, [gpu.wrap_tensor(t) for t in (tx, tq, ts, tg, ty)])
    gpu.sync()
    check(ty.cpu().numpy(), O.gemm_fp4(x, wq, ws, wg))


def test_bounded_wait_reports_and_returns(gpu):
    """A wait on a barrier nothing completes gives up after its limit and sets the status word;
    the context stays usable."""
    assert gpu.status_word() == 0
    gpu.selftest_bounded_wait(limit_us=2000)
    assert gpu.status_word() == L.device.STATUS_WAIT_NEVER
    assert gpu.status_word() == 0                                # reading clears it
    x, wq, ws, wg = inputs.make_case(32, 128, 64, seed_base=5)
    check(L.gemm_fp4(gpu, x, wq, ws, wg), O.gemm_fp4(x, wq, ws, wg))


# ---------------------------------------------------------------- fused all-gather epilogue

@pytest.mark.parametrize("m,n,k,splits", [(512, 256, 512, 1), (300, 384, 2048, 3), (64, 256, 1024, 2)])
def test_gather_epilogue_writes_every_ranks_y(gpu, m, n, k, splits):
    """The n-sharded launch with the all-gather fused in: this 'rank' owns columns [n0, n0+n) of a wider
    y and stores them into every rank's buffer.  Here the 'ranks' are three buffers on one GPU."""
    n_total, n0 = 1024, 384
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=n + k)
    r = inputs.make_residual(m, n, seed_base=3)
    want = O.gemm_fp4(x, wq, ws, wg, r=r)
    q = L.QBuf(gpu, wq, ws, wg)
    xb, rb = gpu.upload(x), gpu.upload(r)
    ys = [gpu.alloc(4 * m * n_total) for _ in range(3)]
    for y in ys:
        gpu.memset(y, 0xFF)
    pipe = gpu.plan_gemm_fp4(m, n, k, residual=True, kernel=3, k_splits=splits)
    gpu.run_gather(pipe, xb, q.wq, q.ws, q.wg, rb, [y.ptr for y in ys], n_total, n0)
    assert gpu.status_word() == 0
    for y in ys:
        full = gpu.download(y, np.float32, (m, n_total))
        check(full[:, n0:n0 + n], want)
        assert np.isnan(full[:, :n0]).all() and np.isnan(full[:, n0 + n:]).all()      # nothing else touched
    with pytest.raises(L.LexbError):
        gpu.run_gather(pipe, xb, q.wq, q.ws, q.wg, rb, [y.ptr for y in ys], n_total, n_total - 128)


# ---------------------------------------------------------------- accuracy against exact arithmetic

def _exact_slice(x, wq, ws, wg, lo, hi):
    """y[:, lo:hi] in f64 from the oracle's own f16 weights: what both implementations approximate."""
    w16 = O.dequant_fp4_f16(wq[lo:hi], ws[lo:hi], wg[lo:hi]).view(np.float16).astype(np.float64)
    return x.astype(np.float64) @ w16.T


def _against_exact(tag, got, oracle, exact):
    """Errors of the GPU result and of the oracle against f64 arithmetic on the same slice; returns the ratio."""
    scale = np.abs(exact).max()
    assert scale > 1e-3
    d_gpu, d_or = got.astype(np.float64) - exact, oracle.astype(np.float64) - exact
    e_gpu, e_or = np.abs(d_gpu).max() / scale, np.abs(d_or).max() / scale
    floor = np.maximum(np.abs(exact), 1e-3 * scale)
    r_gpu, r_or = (np.abs(d_gpu) / floor).max(), (np.abs(d_or) / floor).max()
    # a truncating accumulator loses magnitude: the error is then correlated with the sign of the result
    bias_gpu = float((d_gpu * np.sign(exact)).mean()) / scale
    bias_or = float((d_or * np.sign(exact)).mean()) / scale
    print(f"  {tag}: of scale GPU {e_gpu:.2e} / oracle {e_or:.2e} (x{e_gpu / e_or:.1f}); per element GPU {r_gpu:.2e} / oracle {r_or:.2e}; "
          f"mean signed error toward zero GPU {bias_gpu:+.2e} / oracle {bias_or:+.2e} of scale; rms GPU "
          f"{np.sqrt((d_gpu ** 2).mean()) / scale:.2e} / oracle {np.sqrt((d_or ** 2).mean()) / scale:.2e}")
    return e_gpu, e_or, r_gpu, r_or


# A tensor-core accumulation is not the oracle's: each tcgen05.mma adds its 16 products into the f32 accumulator
# with the low bits cut off rather than rounded to nearest, so every accumulation loses a fraction of a unit in
# the last place of the running sum, always toward zero, where the oracle's round-to-nearest additions err both
# ways and largely cancel.  Measured on the 27B shapes: the GPU result lies 4e-6 to 8e-6 of scale from exact
# arithmetic with a mean signed error of -7e-7 of scale (the bias), the oracle 3e-7 to 8e-7 with none - a
# ratio of 4 to 15 that no schedule of a tensor-core kernel brings to 2, and three decades inside the
# reference's bar for its own GEMM (2e-3 of scale, crates/lex-cuda/tests/device_gpu.rs:294-303).
# The meaningful yardstick on this hardware is the reference's own GPU kernel compiled for it (its wmma GEMM,
# crates/lex-msl/src/gemm.rs:89-320, built by oracle/build_ref.py): this library must be at least as close
# to exact arithmetic as that kernel is.  The ratio to the oracle is kept as a regression bound.
EXACT_OF_SCALE = 2e-5
EXACT_RATIO_TO_ORACLE = 25.0


@pytest.mark.parametrize("m,n,k", [(512, 17408, 5120), (512, 5120, 17408), (2048, 5120, 17408), (256, 17408, 5120),
                                   (512, 2176, 5120), (512, 1024, 2048)])
def test_gpu_error_against_exact_arithmetic(gpu, m, n, k):
    """Distance of the GPU result from f64 arithmetic on the oracle's f16 weights, beside the oracle's own and -
    where an instance of it was built - the reference's own GPU kernel's, on a slice of 256 weight rows: of
    scale, per element, and the mean signed error toward zero."""
    from oracle import refkernels as R
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=17)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    lo, hi = n // 2 - 128, n // 2 + 128
    want = O.gemm_fp4(x, wq, ws, wg, rows=(lo, hi))[:, lo:hi]
    exact = _exact_slice(x, wq, ws, wg, lo, hi)
    e_gpu, e_or, r_gpu, r_or = _against_exact(f"m={m} n={n} k={k}", got[:, lo:hi], want, exact)
    assert e_gpu <= EXACT_OF_SCALE
    assert e_gpu <= EXACT_RATIO_TO_ORACLE * e_or, f"GPU {e_gpu:e} vs oracle {e_or:e} of scale against exact arithmetic"
    for residual in (False, True):
        if R.available(R.gemm_entry(m, n, k, residual)):
            ref = R.gemm(x, wq, ws, wg, np.zeros((m, n), dtype=np.float32) if residual else None)
            e_ref, _, r_ref, _ = _against_exact("  the reference's own kernel (first pair of figures)", ref[:, lo:hi], want, exact)
            assert e_gpu <= e_ref, f"this library {e_gpu:e}, the reference's kernel {e_ref:e} of scale against exact arithmetic"
            break


# ---------------------------------------------------------------- the larger configurations and the shard shapes

def _check_row_slices(got, x, wq, ws, wg, slices, rel_tol, r=None):
    for lo, hi in slices:
        want = O.gemm_fp4(x, wq, ws, wg, r=r, rows=(lo, hi))
        check(got[:, lo:hi], want[:, lo:hi], rel_tol=rel_tol)


def test_gemm_m2048_gate_up_shape(gpu):
    """The 27B MLP prefill at m = 2048 on the gate/up shape (n = 17408, k = 5120): oracle on three slices of rows."""
    n, k = 17408, 5120
    x, wq, ws, wg = inputs.make_case(2048, n, k, seed_base=4)
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    _check_row_slices(got, x, wq, ws, wg, [(0, 128), (n // 2, n // 2 + 128), (n - 128, n)], LONG_K_REL)


@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
def test_gemm_m4096_stack_layer_shapes(gpu, n, k):
    """The calls of the 64-layer stack configuration (m = 4096) on one GPU: oracle on two slices of rows, and the last m tile
    against the same tokens run as a batch of their own with the same tile and no K split (the order of the f32
    additions, and so the bits, belong to the tile shape: the planner may pick another one for 512 tokens alone)."""
    m = 4096
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=6)
    got = L.gemm_fp4(gpu, x, wq, ws, wg, k_splits=1, tm=512)
    _check_row_slices(got, x, wq, ws, wg, [(256, 384), (n - 128, n)], LONG_K_REL)
    sub = L.gemm_fp4(gpu, x[m - 512:].copy(), wq, ws, wg, k_splits=1, tm=512)
    assert np.array_equal(sub, got[m - 512:])


@pytest.mark.parametrize("m", [512, 2048, 4096])
@pytest.mark.parametrize("n,k", [(2176, 5120), (640, 17408), (4352, 5120), (1280, 17408), (8704, 5120), (2560, 17408)])
def test_gemm_shard_shapes_with_the_planned_split(gpu, m, n, k):
    """What one rank of 8, 4 or 2 computes (n/8, n/4, n/2 rows of the 27B MLP matrices) with the K split the
    planner picks for it, against the oracle: the full product for m = 512, slices of rows beyond."""
    x, wq, ws, wg = inputs.make_case(m, n, k, seed_base=n + m)
    pipe = gpu.plan_gemm_fp4(m, n, k)
    d = pipe.describe()
    print(f"  m={m} n={n} k={k}: kernel {d.kernel}, k_splits {d.k_splits}, grid {d.grid}")
    got = L.gemm_fp4(gpu, x, wq, ws, wg)
    if m == 512:
        check(got, O.gemm_fp4(x, wq, ws, wg), rel_tol=LONG_K_REL)
    else:
        _check_row_slices(got, x, wq, ws, wg, [(0, 128), (n - 128, n)], LONG_K_REL)
