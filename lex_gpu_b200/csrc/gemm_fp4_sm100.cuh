// gemm_fp4 for m > 16 on sm_100a:  y[m,n] (f32) = x[m,k] (f16) . dequant(wq, ws, wg)^T (+ r)
//
// The operator is crates/lex-front/lx/gemm_fp4.lx:16-36 (and gemm_fp4_res.lx:10-32 with r);
// the kernel it replaces is the wmma kernel of crates/lex-msl/src/gemm.rs:214-300.
//
// One CTA owns 128 rows of W (one n-tile) and up to 256 tokens (one m-tile) and walks K in
// steps of 64.  The tile is computed transposed: the 128 weight rows are the M side of the
// tcgen05 MMA (A operand), the tokens its N side (B operand), so the accumulator in TMEM
// has one lane per weight row and one column per token.  That keeps a dequant thread's row
// scale in a register and lets token counts from 16 to 256 use one instruction shape.
//
//   warp 8  (one lane)  TMA: x tile [tm tokens x 64 k] f16 -> 128B-swizzled shared memory
//   warps 0-7           dequant: thread (row, half) reads 16 B of codes + its 2 scale bytes
//                       from global memory, decodes 32 weights bit-exactly to f16 and
//                       writes them into the same swizzled K-major layout
//   warp 9  (one lane)  tcgen05.mma kind::f16, 128 x tm x 16, four per stage; tcgen05.commit
//                       frees the stage
//   warps 0-7           epilogue: tcgen05.ld the accumulator, add r, store y (a warp writes
//                       32 consecutive n of one token: 128 contiguous bytes)
#pragma once
#include "fp4_decode.cuh"
#include "sm100_ptx.cuh"

namespace lexb {

constexpr uint32_t GEMM_TN = 128;          // weight rows per CTA (MMA M)
constexpr uint32_t GEMM_BK = 64;           // K per stage: one 128-byte swizzle row of f16
constexpr uint32_t GEMM_DEQ_THREADS = 256;
constexpr uint32_t GEMM_WARP_TMA = 8;
constexpr uint32_t GEMM_WARP_MMA = 9;
constexpr uint32_t GEMM_THREADS = 320;
constexpr uint32_t GEMM_W_TILE_BYTES = GEMM_TN * GEMM_BK * 2;   // 16 KiB

constexpr uint32_t GATHER_MAX = 8;

struct GemmArgs {
    const uint8_t* wq;    // [n, k/2]
    const uint8_t* ws;    // [n, k/16]
    const float* wg;      // [n]
    const float* r;       // [m, n] or null
    float* y;             // [m, n]
    uint32_t* status;     // device status word (ORed)
    unsigned long long* trace;   // null, or 8 counters per CTA written by the two-CTA kernel (phase timers)
    uint32_t m, n, k;
    uint32_t tm;          // tokens per CTA tile: multiple of 16, 16..256
    uint32_t stages;      // pipeline depth (of the x ring in the two-CTA kernel)
    uint32_t w_stages;    // two-CTA kernel: depth of the ring of decoded W tiles
    uint32_t raw_stages;  // two-CTA kernel: depth of the ring of packed-weight blocks (256 K columns each)
    uint32_t k_sub;       // two-CTA kernel: K steps of 64 columns per ring stage (1; 2 only with the W tiles in TMEM)
    uint32_t x_rows;      // two-CTA kernel: tokens each CTA holds of a token block (128; 64 / 32 with tiles of 128 / 64 tokens)
    uint32_t tmem_cols;   // power of two >= max(32, n_acc * tm)
    uint32_t n_acc;       // 1 or 2 accumulators; with 2, even and odd K steps alternate
    uint32_t m_tiles;     // ceil(m / tm)
    uint32_t x_tx_bytes;  // bytes one TMA x tile delivers: min(tm, m) rows of 128 bytes
    uint32_t flags;       // bit 0 (two-CTA kernel): reuse the W tile from the MMA's A collector buffer
    // split-K (two-CTA kernel): split s of k_splits takes K steps [s * kb_per_split, ...) and writes its
    // partial product to partial[s][m][n]; a reduction kernel then forms y.  k_splits = 1: y is written.
    uint32_t k_splits, kb_per_split;
    // Fused all-gather (two-CTA kernel): with gather_world > 0 the result is not written to y but to
    // column gather_n0 + j of every gather_y[d], d < gather_world - y buffers of row length gather_n, one
    // per GPU, mapped into this GPU's address space (plain peer stores over NVLink; no copy-engine loads).
    float* gather_y[GATHER_MAX];
    uint32_t gather_world, gather_n, gather_n0;
    uint32_t tok_blocks;  // two-CTA kernel: 256-token blocks per tile, 2 (m > 256) or 1; with 1, TMEM holds two
                          // accumulators that take even and odd K steps
    float* partial;
    // Two-CTA kernel, gate/up fused (crates/lex-rt/src/qwen_run.rs:3165-3183): the weight rows are gate and up
    // interleaved (row 2j = gate j, row 2j + 1 = up j) and, with `act` set (or `silu_gather` with the gather
    // pointers), the epilogue writes silu(gate) * up as f16 [m, n/2] - the activation `down` reads - instead of
    // the f32 y [m, n].
    uint16_t* act;
    uint32_t silu_gather;
};

// silu(g) * u = g * (1 / (1 + exp(-g))) * u in f32, one rounding per operation, as the interpreter evaluates
// lex_front::llama::silu_mul (crates/lex-front/src/llama.rs:879-888; sigmoid: crates/lex-front/src/ir.rs:244)
__device__ __forceinline__ float silu_mul_f32(float g, float u) {
    const float sg = __frcp_rn(__fadd_rn(1.0f, expf(-g)));      // 1 / x rounded to nearest: the same bits as the division
    return __fmul_rn(__fmul_rn(g, sg), u);
}
__device__ __forceinline__ uint16_t f32_to_f16_bits(float v) {
    uint16_t h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
    return h;
}

__host__ __device__ constexpr uint32_t gemm_stage_bytes(uint32_t tm) { return tm * 128u + GEMM_W_TILE_BYTES; }
// stages, then 3 barriers per stage + 1, the TMEM slot and the abort flag; 1 KiB alignment slack
__host__ __device__ constexpr uint32_t gemm_smem_bytes(uint32_t tm, uint32_t stages) {
    return stages * gemm_stage_bytes(tm) + (3u * stages + 1u) * 8u + 16u + 1024u;
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_fp4_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;          // swizzled tiles need 1 KiB alignment
    uint8_t* const smem = smem_raw + (base - raw_addr);

    const uint32_t S = a.stages;
    const uint32_t x_bytes = a.tm * 128u;
    const uint32_t stage_bytes = x_bytes + GEMM_W_TILE_BYTES;
    const uint32_t bars = base + S * stage_bytes;               // shared-space address of barrier 0
    auto x_full = [&](uint32_t s) { return bars + 8u * s; };
    auto w_full = [&](uint32_t s) { return bars + 8u * (S + s); };
    auto empty = [&](uint32_t s) { return bars + 8u * (2u * S + s); };
    const uint32_t acc_full = bars + 8u * 3u * S;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(smem + S * stage_bytes + (3u * S + 1u) * 8u);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t m_tile = blockIdx.x % a.m_tiles, n_tile = blockIdx.x / a.m_tiles;
    const uint32_t m0 = m_tile * a.tm, n0 = n_tile * GEMM_TN;
    const uint32_t KB = a.k / GEMM_BK;

    if (tid == 0) {
        *abort_flag = 0;
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(x_full(s), 1);
            mbar_init(w_full(s), GEMM_DEQ_THREADS / 32u);   // one arrival per dequant warp
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
    }
    if (warp == GEMM_WARP_TMA && lane == 0) prefetch_tensormap(&tmap_x);
    if (warp == GEMM_WARP_MMA) {
        tmem_alloc(smem_u32(tmem_slot), a.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == GEMM_WARP_TMA) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t issued = 0;
            bool ok = true;
            RingPos pp;
            for (uint32_t kb = 0; kb < KB && ok; kb++, pp.advance(S)) {
                const uint32_t s = pp.s, ph = pp.ph;
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(x_full(s), a.x_tx_bytes);
                tma_load_2d(base + s * stage_bytes, &tmap_x, (int)(kb * GEMM_BK), (int)m0, x_full(s));
                issued = kb + 1;
            }
            if (!ok || *abort_flag) {
                // leave only after this thread's own copies have landed (bounded)
                const uint32_t first = issued > S ? issued - S : 0;
                for (uint32_t kb = first; kb < issued; kb++) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(x_full(kb % S), (kb / S) & 1u)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicOr(a.status, ST_WAIT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == GEMM_WARP_MMA) {
        // ---------------------------------------------------------------- MMA issuer
        // The whole warp runs the loop with warp-uniform values; one elected lane issues.
        {
            const uint32_t idesc = umma_idesc_f16_f32(GEMM_TN, a.tm);
            const uint32_t x_lo0 = umma_desc_lo(base), stage16 = stage_bytes >> 4, w_off16 = x_bytes >> 4;
            bool ok = true;
            RingPos pp;
            uint32_t acc_sel = 0;                        // which accumulator takes this K step
            for (uint32_t kb = 0; kb < KB; kb++, pp.advance(S)) {
                const uint32_t s = pp.s, ph = pp.ph;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(x_full(s), ph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_X_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(w_full(s), ph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_W_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t b_lo = x_lo0 + s * stage16, a_lo = b_lo + w_off16;
                // Two accumulators halve the run of truncating f32 additions each one sees (the
                // tensor core does not round to nearest when it accumulates).
                const uint32_t d = tmem_base + acc_sel * a.tm;
                if (++acc_sel == a.n_acc) acc_sel = 0;
                if (elect_one()) {
                    umma1_flag(d, a_lo, b_lo, idesc, kb >= a.n_acc);
#pragma unroll
                    for (uint32_t kk = 1; kk < GEMM_BK / 16; kk++) umma1_acc(d, a_lo + 2u * kk, b_lo + 2u * kk, idesc);
                    umma_commit(empty(s));      // frees the stage once these MMAs have read it
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit(acc_full);  // accumulator complete
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- dequant warps 0-7
        // Thread (row r, half h): a warp covers 32 consecutive rows and one half, so the eight
        // 16-byte chunks any 8 consecutive lanes store fall into eight different bank groups.
        const uint32_t r = tid & 127u, h = tid >> 7;
        const uint32_t row = n0 + r;
        const float g = __ldg(a.wg + row);
        const uint4* qrow = reinterpret_cast<const uint4*>(a.wq + (size_t)row * (a.k / 2)) + h;
        const uint32_t* srow = reinterpret_cast<const uint32_t*>(a.ws + (size_t)row * (a.k / 16));
        const uint32_t w_off = r * 128u;
        const uint32_t sw_xor = r & 7u;
        // two K steps of codes and scales in flight
        uint4 q0 = __ldg(qrow), q1 = KB > 1 ? __ldg(qrow + 2) : make_uint4(0, 0, 0, 0);
        uint32_t s0 = __ldg(srow), s1 = KB > 1 ? __ldg(srow + 1) : 0u;
        bool ok = true;
        RingPos pp;
        for (uint32_t kb = 0; kb < KB; kb++, pp.advance(S)) {
            const uint32_t s = pp.s, ph = pp.ph;
            const uint4 q = q0;
            const uint32_t sw = s0 >> (16u * h);
            q0 = q1;
            s0 = s1;
            if (kb + 2 < KB) {
                q1 = __ldg(qrow + 2u * (kb + 2));
                s1 = __ldg(srow + kb + 2);
            }
            uint4 o0, o1, o2, o3;
            decode_group16(make_uint2(q.x, q.y), sw & 0xFFu, g, o0, o1);
            decode_group16(make_uint2(q.z, q.w), (sw >> 8) & 0xFFu, g, o2, o3);
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty(s), ph ^ 1u, abort_flag))) {   // warp-uniform give-up
                atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                *abort_flag = 1;
                ok = false;
                break;
            }
            uint8_t* wt = smem + s * stage_bytes + x_bytes + w_off;
            const uint32_t c = 4u * h;
            *reinterpret_cast<uint4*>(wt + (((c + 0u) ^ sw_xor) << 4)) = o0;
            *reinterpret_cast<uint4*>(wt + (((c + 1u) ^ sw_xor) << 4)) = o1;
            *reinterpret_cast<uint4*>(wt + (((c + 2u) ^ sw_xor) << 4)) = o2;
            *reinterpret_cast<uint4*>(wt + (((c + 3u) ^ sw_xor) << 4)) = o3;
            fence_proxy_async_smem();       // make the generic-proxy stores visible to the MMA
            __syncwarp();                   // one arrival per warp: arrivals on one barrier serialise
            if (lane == 0) mbar_arrive(w_full(s));
        }
        __syncwarp();
        // ---------------------------------------------------------------- epilogue
        uint32_t go = 0;
        if (lane == 0) {
            go = ok && mbar_wait(acc_full, 0, abort_flag);
            if (!go) {
                atomicOr(a.status, ST_WAIT_ACC);
                *abort_flag = 1;
            }
        }
        go = __shfl_sync(0xFFFFFFFFu, go, 0);
        if (go) {
            tc_fence_after_sync();
            const uint32_t quarter = warp & 3u, half = warp >> 2;
            const uint32_t out_row = n0 + 32u * quarter + lane;
            const uint32_t chunks = a.tm / 16u;
            for (uint32_t c = half; c < chunks; c += 2u) {
                uint32_t v[16];
                tmem_ld_32x32b_x16(tmem_base + ((32u * quarter) << 16) + c * 16u, v);
                if (a.n_acc > 1 && KB > 1) {
                    uint32_t v2[16];
                    tmem_ld_32x32b_x16(tmem_base + ((32u * quarter) << 16) + a.tm + c * 16u, v2);
                    tmem_ld_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 16; j++)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
                } else {
                    tmem_ld_wait();
                }
                const uint32_t t0 = m0 + c * 16u;
#pragma unroll
                for (uint32_t j = 0; j < 16; j++) {
                    const uint32_t t = t0 + j;
                    if (t < a.m) {
                        const size_t o = (size_t)t * a.n + out_row;
                        float val = __uint_as_float(v[j]);
                        if (a.r) val = val + __ldg(a.r + o);
                        a.y[o] = val;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == GEMM_WARP_MMA) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, a.tmem_cols);
    }
}

}  // namespace lexb
