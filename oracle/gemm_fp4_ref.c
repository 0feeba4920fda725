/* CPU restatement of lex's reference interpreter for the one operator `gemm_fp4`
 * (and its residual twin `gemm_fp4_res`).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed CPU
 * baseline.  The product library never links, loads or calls it.
 *
 * Parity status: the reference keeps no stored output vectors for this
 * operator; its tests recompute expected values from an independent f64
 * restatement (crates/lex-front/tests/syntax.rs:509-585, 634-683).  This oracle
 * is pinned against those known-answer recipes (same inputs, same tolerance)
 * and against exhaustive decode tables; the f16 bit patterns of the staged
 * weights are pinned by IEEE-754 round-to-nearest-even only ("parity unpinned"
 * by any reference fixture for individual f16 bits).
 *
 * What is followed, with the reference lines:
 *   e2m1            crates/lex-front/src/interp.rs:30-34
 *   e4m3            crates/lex-front/src/interp.rs:37-47   (OCP e4m3fn, NaN at 0x7f/0xff)
 *   round(F16)      crates/lex-front/src/interp.rs:76-82   (half 2.7.1 f16::from_f32: RN-even)
 *   load rounding   crates/lex-front/src/interp.rs:360-374
 *   dequant_fp4     crates/lex-front/src/interp.rs:643-657 (low nibble = even column,
 *                   left-to-right f32 product  (e2m1 * e4m3) * wg)
 *   stage f16       crates/lex-front/src/interp.rs:500-507
 *   mma             crates/lex-front/src/interp.rs:508-526 (per K-tile: s = 0; s += a*b
 *                   sequentially in f32; acc += s)
 *   add_window      crates/lex-front/src/interp.rs:485-499 (acc + r, f32)
 *   store           crates/lex-front/src/interp.rs:465-479 (f32: identity)
 *   loop structure  crates/lex-front/lx/gemm_fp4.lx:16-39  (Ada schedule bk = 64)
 *   metrics         crates/lex-ir/src/reference.rs:69-82, crates/lex-cuda/tests/device_gpu.rs:294-303
 *
 * Build with -ffp-contract=off: the interpreter multiplies and adds separately.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LEXO_API __attribute__((visibility("default")))

/* ---- scalar formats --------------------------------------------------- */

/* interp.rs:30-34 */
LEXO_API float lexo_e2m1(uint8_t code) {
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = mag[code & 7];
    return (code & 8) ? -v : v;
}

/* interp.rs:37-47 */
LEXO_API float lexo_e4m3(uint8_t b) {
    int e = (b >> 3) & 0xF;
    float m = (float)(b & 7);
    float v;
    if (e == 0)
        v = m * ldexpf(1.0f, -9);
    else if (e == 15 && (b & 7) == 7)
        v = NAN;
    else
        v = (1.0f + m / 8.0f) * ldexpf(1.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary32 -> binary16, round to nearest even, subnormals kept,
 * overflow to infinity, NaN stays NaN (quiet, sign kept): the behaviour of
 * half 2.7.1 `f16::from_f32` that interp.rs:79 relies on. */
LEXO_API uint16_t lexo_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ex = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (ex == 0xFF) {                       /* inf / NaN */
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7E00u | (man >> 13));
    }
    int32_t e = (int32_t)ex - 127 + 15;     /* rebias */
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);            /* overflow */
    if (e <= 0) {                           /* f16 subnormal or zero */
        if (e < -10) return (uint16_t)sign; /* below half of the smallest subnormal */
        man |= 0x800000u;                   /* implicit one */
        uint32_t shift = (uint32_t)(14 - e);            /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);             /* a carry lands in exponent 1 */
    }
    uint32_t half = (uint32_t)(e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;  /* carry may reach inf */
    return (uint16_t)(sign | half);
}

LEXO_API float lexo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t ex = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (ex == 0) {
        if (man == 0) return bits_f32(sign);
        float v = (float)man * ldexpf(1.0f, -24);
        return (sign ? -v : v);
    }
    if (ex == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((ex + 112u) << 23) | (man << 13));
}

/* ---- dequant ---------------------------------------------------------- */

/* One staged weight as the interpreter forms it: interp.rs:648-653 then :500-507.
 * `byte` is the packed byte, `col` the logical column (parity picks the nibble). */
static inline float dequant_one(uint8_t byte, int col, uint8_t sbyte, float g) {
    uint8_t code = (col % 2 == 0) ? (uint8_t)(byte & 0xF) : (uint8_t)(byte >> 4);
    float scale = lexo_e4m3(sbyte);
    float w = lexo_e2m1(code) * scale;   /* exact: at most 6 significant bits */
    w = w * g;                           /* f32 rounding */
    return w;
}

/* f16 bit patterns of every staged weight, row-major [n, k]. */
LEXO_API void lexo_dequant_fp4_f16(uint32_t n, uint32_t k, const uint8_t* wq, const uint8_t* ws,
                                   const float* wg, uint16_t* w16) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < (int64_t)n; j++) {
        const uint8_t* q = wq + (size_t)j * (k / 2);
        const uint8_t* s = ws + (size_t)j * (k / 16);
        for (uint32_t p = 0; p < k; p++)
            w16[(size_t)j * k + p] = lexo_f32_to_f16(dequant_one(q[p / 2], (int)p, s[p / 16], wg[j]));
    }
}

/* ---- the operator ------------------------------------------------------ */

/* y[m,n] = x[m,k] . dequant(wq,ws,wg)^T (+ r).  x is given as f16 bit patterns.
 * bk is the K-tile of the schedule (64 for nvidia-ada, 32 for apple-m-series):
 * products are summed sequentially within a tile and the tile sum is then added
 * to the accumulator, exactly as Op::Mma inside the `for p` loop does.
 * Rows [n0, n1) of W only (n0 = 0, n1 = n for the whole operator): the timed
 * baseline uses row slices.  Returns 0, or -1 on a shape the .lx program rejects
 * (crates/lex-front/src/syntax.rs:1513-1516 "does not divide"). */
LEXO_API int lexo_gemm_fp4_rows(uint32_t m, uint32_t n, uint32_t k, uint32_t bk, const uint16_t* x16,
                                const uint8_t* wq, const uint8_t* ws, const float* wg, const float* r,
                                float* y, uint32_t n0, uint32_t n1, int threads) {
    enum { JB = 4, IC = 64 };
    if (bk == 0 || k % bk != 0 || bk % 16 != 0 || k % 16 != 0 || n1 > n || n0 > n1) return -1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    /* x as f32, transposed to [k][m]: the token index becomes the contiguous one, so the
     * compiler may vectorise ACROSS tokens.  Each y element still sees exactly the
     * interpreter's order: products summed one by one within a K-tile, tile sums added
     * one by one into the accumulator. */
    float* xt = (float*)__builtin_malloc((size_t)m * k * sizeof(float));
    if (!xt) return -2;
    for (uint32_t i = 0; i < m; i++)
        for (uint32_t p = 0; p < k; p++) xt[(size_t)p * m + i] = lexo_f16_to_f32(x16[(size_t)i * k + p]);
    int rc = 0;
    int64_t nblocks = ((int64_t)(n1 - n0) + JB - 1) / JB;
#pragma omp parallel
    {
        float* w = (float*)__builtin_malloc((size_t)JB * k * sizeof(float));
        if (!w) {
#pragma omp atomic write
            rc = -2;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (int64_t b = 0; b < nblocks; b++) {
                uint32_t j0 = n0 + (uint32_t)b * JB;
                uint32_t nj = (n1 - j0 < JB) ? (n1 - j0) : JB;
                for (uint32_t jb = 0; jb < nj; jb++) { /* dequant_fp4, then stage f16 */
                    uint32_t j = j0 + jb;
                    const uint8_t* q = wq + (size_t)j * (k / 2);
                    const uint8_t* s = ws + (size_t)j * (k / 16);
                    for (uint32_t p = 0; p < k; p++)
                        w[(size_t)jb * k + p] = lexo_f16_to_f32(
                            lexo_f32_to_f16(dequant_one(q[p / 2], (int)p, s[p / 16], wg[j])));
                }
                for (uint32_t i0 = 0; i0 < m; i0 += IC) {
                    uint32_t ni = (m - i0 < IC) ? (m - i0) : IC;
                    float acc[JB][IC], sum[JB][IC];
                    for (uint32_t jb = 0; jb < JB; jb++)
                        for (uint32_t i = 0; i < IC; i++) acc[jb][i] = 0.0f;
                    for (uint32_t t = 0; t < k; t += bk) {
                        for (uint32_t jb = 0; jb < JB; jb++)
                            for (uint32_t i = 0; i < IC; i++) sum[jb][i] = 0.0f;
                        for (uint32_t p = t; p < t + bk; p++) {
                            const float* xp = xt + (size_t)p * m + i0;
                            for (uint32_t jb = 0; jb < nj; jb++) {
                                float wv = w[(size_t)jb * k + p];
                                for (uint32_t i = 0; i < ni; i++) sum[jb][i] += xp[i] * wv;
                            }
                        }
                        for (uint32_t jb = 0; jb < nj; jb++)
                            for (uint32_t i = 0; i < ni; i++) acc[jb][i] += sum[jb][i];
                    }
                    for (uint32_t jb = 0; jb < nj; jb++)
                        for (uint32_t i = 0; i < ni; i++) {
                            size_t o = (size_t)(i0 + i) * n + (size_t)(j0 + jb);
                            float v = acc[jb][i];
                            if (r) v = v + r[o]; /* add_window */
                            y[o] = v;
                        }
                }
            }
        }
        __builtin_free(w);
    }
    __builtin_free(xt);
    return rc;
}

LEXO_API int lexo_gemm_fp4(uint32_t m, uint32_t n, uint32_t k, uint32_t bk, const uint16_t* x16,
                           const uint8_t* wq, const uint8_t* ws, const float* wg, const float* r, float* y,
                           int threads) {
    return lexo_gemm_fp4_rows(m, n, k, bk, x16, wq, ws, wg, r, y, 0, n, threads);
}

/* ---- matmul_q_x with the NVFP4 layout ------------------------------------ */

/* crates/lex-front/src/llama.rs:444-499: per chunk of kc columns, part = MatMulNT(x, w) with
 * w = DequantFp4 (f32, NOT rounded to f16: interp.rs:643-657) and a sequential f32 sum
 * (interp.rs:527-548); acc += part; y = acc (+ r).  The runtime calls it with kc = n_in
 * (crates/lex-rt/src/qwen_run.rs:2605).  x is given as f32 values (an f16 x is widened by
 * the caller, which is exact).  Returns 0, or -1 when kc does not divide k or is not whole
 * groups of 16 (llama.rs:407-413). */
LEXO_API int lexo_matmul_q_x(uint32_t m, uint32_t n, uint32_t k, uint32_t kc, const float* x,
                             const uint8_t* wq, const uint8_t* ws, const float* wg, const float* r,
                             float* y, int threads) {
    if (kc == 0 || k % kc != 0 || kc % 16 != 0) return -1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    int rc = 0;
#pragma omp parallel
    {
        float* w = (float*)__builtin_malloc((size_t)k * sizeof(float));
        if (!w) {
#pragma omp atomic write
            rc = -2;
        } else {
#pragma omp for schedule(static)
            for (int64_t j = 0; j < (int64_t)n; j++) {
                const uint8_t* q = wq + (size_t)j * (k / 2);
                const uint8_t* s = ws + (size_t)j * (k / 16);
                for (uint32_t p = 0; p < k; p++) w[p] = dequant_one(q[p / 2], (int)p, s[p / 16], wg[j]);
                for (uint32_t i = 0; i < m; i++) {
                    const float* xi = x + (size_t)i * k;
                    float acc = 0.0f;
                    for (uint32_t c = 0; c < k; c += kc) {
                        float part = 0.0f;
                        for (uint32_t p = c; p < c + kc; p++) part += xi[p] * w[p];
                        acc += part;
                    }
                    size_t o = (size_t)i * n + (size_t)j;
                    if (r) acc = acc + r[o];
                    y[o] = acc;
                }
            }
        }
        __builtin_free(w);
    }
    return rc;
}

/* ---- metrics ----------------------------------------------------------- */

/* crates/lex-ir/src/reference.rs:69-82 */
LEXO_API float lexo_max_rel_err(const float* got, const float* want, size_t len) {
    float worst = 0.0f;
    for (size_t i = 0; i < len; i++) {
        float g = got[i], w = want[i];
        if (!isfinite(g) || !isfinite(w)) return INFINITY;
        float err = fabsf(g - w) / fmaxf(fabsf(w), 1e-3f);
        if (err > worst) worst = err;
    }
    return worst;
}

/* crates/lex-cuda/tests/device_gpu.rs:294-303: max|got-want| / max|want|.
 * out[0] = error of scale, out[1] = scale (the caller asserts scale > 1e-3),
 * out[2] = per-element relative error with a floor of 1e-3 * scale. */
LEXO_API void lexo_err_of_scale(const float* got, const float* want, size_t len, double* out) {
    double scale = 1e-6, worst = 0.0;
    for (size_t i = 0; i < len; i++) {
        double a = fabs((double)want[i]);
        if (a > scale) scale = a;
    }
    double floor_ = 1e-3 * scale, worst_rel = 0.0;
    for (size_t i = 0; i < len; i++) {
        double d = fabs((double)got[i] - (double)want[i]);
        if (!(d == d)) d = INFINITY;
        if (d > worst) worst = d;
        double den = fabs((double)want[i]);
        if (den < floor_) den = floor_;
        if (d / den > worst_rel) worst_rel = d / den;
    }
    out[0] = worst / scale;
    out[1] = scale;
    out[2] = worst_rel;
}

LEXO_API int lexo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
