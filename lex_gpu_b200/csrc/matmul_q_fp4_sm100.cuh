// matmul_q (NVFP4 layout) for a few tokens on the block-scaled FP4 tensor-core path of sm_100a.
//
//     y[t, j] = wg[j] * sum_g e4m3(ws[j, g]) * sum_{p in group g} e2m1(wq[j, p]) * x[t, p]   (+ r[t, j])
//
// which is lex's `matmul_q_x` with the NVFP4 layout (crates/lex-front/src/llama.rs:444-499, weights
// dequantised by `Op::DequantFp4`, crates/lex-front/src/interp.rs:643-657) with the row scale
// factored out of the sum: the weights are NOT rounded to f16 here, unlike in `gemm_fp4`.  This is
// the operator the model runs for decode and for speculative verification (t <= 8,
// crates/lex-rt/src/qwen_run.rs:2605-2606).
//
// The tensor core does the whole decode: `tcgen05.mma.kind::mxf4nvf4.block_scale` multiplies packed
// E2M1 codes by a UE4M3 scale per 16 values of K, which is exactly how wq and ws are stored.  The
// packed codes go from global memory to shared memory by TMA and are never touched by a thread; the
// integer pipe, which bounds the table-lookup decode of `matvec_fp4_kernel`, is idle here and the
// kernel streams at memory speed.
//
// The activations have to be E2M1 as well.  Each token (f16, or f32) is split into MQ_PIECES = 8 rows of
// 2-bit digits: inside a group of 16 values with largest exponent E, a value is sign * I * 2^(E-15) with a
// 16-bit integer I = round(|x| * 2^(15-E)).  For f16 input that is exact for every value within 2^5 of the
// group's maximum (11 significant bits fit with 5 to spare) and finer than f16's own grid there; f32 input
// keeps 16 bits below the group's maximum, which is what the reference's own integer path keeps
// (`quant16`, crates/lex-msl/src/int8.rs:44-99).  I = sum_p digit_p * 4^(7-p); piece p holds the E2M1 codes
// of digit_p / 2 (0, 0.5, 1, 1.5 are codes 0..3) and the group scale 2^(E - 2p - G), G a per-token offset
// that keeps the scales inside UE4M3's range; the epilogue adds the 8 accumulator columns of a token and
// multiplies by 2^G * wg[j].  So a token costs 8 columns of N, the minimum N of the instruction anyway.
// Groups (and tokens) whose largest magnitude is below 2^-111 count as zero.
//
// Scale bytes with the sign bit set are legal E4M3 (the reference decodes them as negative scales):
// the hardware scale is unsigned, so the sign is moved into the 16 codes of the group in shared
// memory.  The two NaN bytes (0x7f, 0xff) make the whole output row NaN, as in the reference.
//
// Block = 128 weight rows (one row tile) x one K range.  Warp 0 issues the TMA loads (codes per 256 of K
// into a ring of stages, raw scale bytes per 1024 of K into a ring of their own, one group ahead); warp 1
// copies each stage's scale blocks into tensor memory and issues its 4 MMAs of K = 64, alternating two
// accumulators; warps 2-5 and 6-9 re-lay the weight scales of the even and the odd stages into the
// 32 x 16-byte blocks the instruction reads (warps 2-5 then run the epilogue); warps 10-17 derive the
// tokens' digit rows - unless matmul_q_pieces_kernel has done that once for the launch (PRE: from 5 tokens
// on), in which case warp 0 loads them with the weights.  With K split over blocks, the last block of a
// row tile to finish sums the partial products.  Every wait is bounded.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace lexb {

constexpr uint32_t MQ_ROWS = 128;                         // weight rows per block
constexpr uint32_t MQ_STAGE_K = 256;                      // values of K per stage: one 128-byte row of codes
constexpr uint32_t MQ_PIECES = 8;                         // E2M1 digit rows per token
constexpr uint32_t MQ_MAX_TOKENS = 32;
constexpr uint32_t MQ_CODE_BYTES = MQ_ROWS * 128u;        // packed codes of a stage
// the tokens' pieces of a stage: 128 bytes x 8 rows per token, room for 4, 8, 16 or 32 tokens
__host__ __device__ constexpr uint32_t matmul_q_b_bytes(uint32_t m) {
    return m <= 4u ? 4096u : (m <= 8u ? 8192u : (m <= 16u ? 16384u : 32768u));
}
constexpr uint32_t MQ_SF_BYTES = 4u * 512u;               // scale blocks of A for a stage: one 512-byte block per MMA
// ... of B: one block per MMA covers 128 rows of B (16 tokens), so more than 16 tokens take two
__host__ __device__ constexpr uint32_t matmul_q_sfb_bytes(uint32_t m) { return m <= 16u ? 2048u : 4096u; }
__host__ __device__ constexpr uint32_t matmul_q_stage_bytes(uint32_t m) {
    // a multiple of 1024: stages start on a swizzle-pattern boundary
    return MQ_CODE_BYTES + matmul_q_b_bytes(m) + MQ_SF_BYTES + matmul_q_sfb_bytes(m);
}
// The scale bytes as stored come in their own, coarser ring: one load covers MQ_WS_GROUP stages, so
// that a row's piece of it is 64 bytes (16 bytes per stage would fetch half-used 32-byte sectors).
constexpr uint32_t MQ_WS_GROUP = 4;
constexpr uint32_t MQ_WS_SLOTS = 3;
constexpr uint32_t MQ_WS_SLOT_BYTES = MQ_ROWS * 16u * MQ_WS_GROUP;
constexpr uint32_t MQ_SCALE_WARPS = 8;                    // warps 2-5: weight scales of even stages, then the epilogue;
                                                          // warps 6-9: weight scales of odd stages
constexpr uint32_t MQ_PIECE_WARPS = 8;                    // warps 10-17: the tokens' digit rows
constexpr uint32_t MQ_THREADS = 32u * (2u + MQ_SCALE_WARPS + MQ_PIECE_WARPS);
constexpr uint32_t MQ_TMEM_COLS = 512;
constexpr uint32_t MQ_MAX_STAGES = 8;
// Tensor memory.  Up to 16 tokens (N <= 128): two accumulators at columns 0 and 128 that take the even and the
// odd stages, the scale rings of A and B at 256 and 384, 16 columns per stage.  17-32 tokens (N <= 256): one
// accumulator, A's ring at 256 (at most 4 stages), B's at 320 with 32 columns per stage.
constexpr uint32_t MQ_TMEM_D1 = 128;
constexpr uint32_t MQ_TMEM_SFA = 256;
constexpr uint32_t MQ_TMEM_SFB = MQ_TMEM_SFA + 16u * MQ_MAX_STAGES;
constexpr uint32_t MQ_TMEM_SFB_WIDE = 320;
constexpr uint32_t MQ_WIDE_MAX_STAGES = 4;

struct MatmulQArgs {
    const void* x;           // [m, k], f16 or f32
    const float* wg;         // [n]
    const float* r;          // [m, n] or null
    float* y;                // [m, n]
    float* partial;          // [k_splits][m][n] when k_splits > 1
    uint32_t* counters;      // [n / 128], zero between launches: how many splits of a row tile have stored their partial
    uint32_t* status;
    unsigned long long* trace;   // 16 phase timers per block, or null
    uint32_t m, n, k, stages;
    uint32_t k_splits, kb_per_split;   // in stages of 256
    uint32_t ws_pitch;                 // bytes per row of a scale load: min(64, k / 16)
    uint32_t flags;                    // bit 0: the weights are constant, load them before the launch ahead has finished
    // The launch that follows this one in the step list, when it is of this kernel too (grid 0: none): its
    // blocks' first `next_stages` stages of weights are prefetched into L2 by this launch's blocks once
    // they have requested all of their own, so that DRAM keeps streaming through this launch's tail and the
    // next one's set-up instead of idling.
    uint32_t next_grid, next_k_splits, next_kb_per_split, next_kb_all, next_stages, next_ws_pitch;
    // PRE variant: the tokens' digit rows come from matmul_q_pieces_kernel (once per launch instead of
    // once per block): scale blocks of B as the stages want them, [k / 256][2048] bytes, and the tokens'
    // largest magnitudes as f32 bits; the digit rows themselves arrive through their own tensor map.
    const uint8_t* pre_sfb;
    const uint32_t* pre_amax;
};

__host__ __device__ constexpr uint32_t matmul_q_smem_bytes(uint32_t m, uint32_t stages) {
    return stages * matmul_q_stage_bytes(m) + MQ_WS_SLOTS * MQ_WS_SLOT_BYTES + (3u * stages + 1u + 2u * MQ_WS_SLOTS) * 8u + 192u + MQ_ROWS + 1024u;
}

// bits [2i+1 : 2i] of an 8-bit value -> byte i
__device__ __forceinline__ uint32_t mq_spread8(uint32_t t) {
    uint32_t u = (t | (t << 12)) & 0x000F000Fu;
    return (u | (u << 6)) & 0x03030303u;
}

// UE4M3 byte of 2^q (0 when it is below the smallest subnormal)
__device__ __forceinline__ uint32_t mq_ue4m3_pow2(int q) {
    if (q >= -6) return static_cast<uint32_t>(q + 7) << 3;
    if (q >= -9) return 1u << (q + 9);
    return 0u;
}

// One lane's 8 consecutive values of K (f32 bit patterns) -> for each of the 8 pieces the 4 bytes that hold
// this lane's 8 codes (two per byte, even K low), and the exponent field of the largest magnitude of the
// group of 16 the lane shares with its neighbour (lanes 2g, 2g+1).  Whole warp.
__device__ __forceinline__ void mq_digits(const uint32_t (&fb)[8], uint32_t (&w)[8], uint32_t& e8) {
    uint32_t am = 0;
#pragma unroll
    for (uint32_t i = 0; i < 8; i++) am = max(am, fb[i] & 0x7FFFFFFFu);
    am = max(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
    // |x| = I * 2^(E - 15), E the group's largest exponent: I = |x| * 2^(142 - e8), 16 bits.  Groups
    // below 2^-111 count as zero (their scale factor would leave f32's range).
    e8 = am >> 23;
    const float to_fixed = e8 >= 16u ? __uint_as_float((269u - e8) << 23) : 0.0f;
    uint32_t blo[4], bhi[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; i++) {
        const uint32_t b0 = fb[2 * i], b1 = fb[2 * i + 1];
        const uint32_t i0 = min(__float2uint_rn(__uint_as_float(b0 & 0x7FFFFFFFu) * to_fixed), 65535u);
        const uint32_t i1 = min(__float2uint_rn(__uint_as_float(b1 & 0x7FFFFFFFu) * to_fixed), 65535u);
        const uint32_t sg = ((0u - (b0 >> 31)) & 0x08080808u) | ((0u - (b1 >> 31)) & 0x80808080u);
        blo[i] = mq_spread8(i0 & 0xFFu) | (mq_spread8(i1 & 0xFFu) << 4) | sg;
        bhi[i] = mq_spread8(i0 >> 8) | (mq_spread8(i1 >> 8) << 4) | sg;
    }
    // byte b of blo[i] / bhi[i] is the code pair of piece 7-b / 3-b: transpose 4x4 bytes
    const uint32_t t0 = __byte_perm(blo[0], blo[1], 0x5140), t1 = __byte_perm(blo[2], blo[3], 0x5140);
    const uint32_t t2 = __byte_perm(blo[0], blo[1], 0x7362), t3 = __byte_perm(blo[2], blo[3], 0x7362);
    w[7] = __byte_perm(t0, t1, 0x5410);
    w[6] = __byte_perm(t0, t1, 0x7632);
    w[5] = __byte_perm(t2, t3, 0x5410);
    w[4] = __byte_perm(t2, t3, 0x7632);
    const uint32_t u0 = __byte_perm(bhi[0], bhi[1], 0x5140), u1 = __byte_perm(bhi[2], bhi[3], 0x5140);
    const uint32_t u2 = __byte_perm(bhi[0], bhi[1], 0x7362), u3 = __byte_perm(bhi[2], bhi[3], 0x7362);
    w[3] = __byte_perm(u0, u1, 0x5410);
    w[2] = __byte_perm(u0, u1, 0x7632);
    w[1] = __byte_perm(u2, u3, 0x5410);
    w[0] = __byte_perm(u2, u3, 0x7632);
}

// 8 halves (one uint4) or 8 floats (two) -> f32 bit patterns
template <bool XF32>
__device__ __forceinline__ void mq_widen(const uint4& lo, const uint4& hi, uint32_t (&fb)[8]) {
    if (XF32) {
        fb[0] = lo.x; fb[1] = lo.y; fb[2] = lo.z; fb[3] = lo.w;
        fb[4] = hi.x; fb[5] = hi.y; fb[6] = hi.z; fb[7] = hi.w;
    } else {
        const uint32_t hw[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[i]));
            fb[2 * i] = __float_as_uint(f.x);
            fb[2 * i + 1] = __float_as_uint(f.y);
        }
    }
}

// offset of the scale byte of (row n of B, group of 16 `grp` of the stage) inside the stage's 2048 bytes:
// one 512-byte block per MMA (4 groups), in it 16 bytes per (n % 32), 4 per (n / 32), one per group
// (with more than 128 rows of B - `wide` - an MMA has two such blocks, rows 0-127 and 128-255)
__device__ __forceinline__ uint32_t mq_sfb_offset(uint32_t n, uint32_t grp, bool wide) {
    return (grp >> 2) * (wide ? 1024u : 512u) + (n >> 7) * 512u + (n & 31u) * 16u + ((n >> 5) & 3u) * 4u + (grp & 3u);
}

// PRE = false: 576 threads, piece warps 10-17 derive the tokens' digit rows in every block (no second launch:
// best for up to 4 tokens).  PRE = true: 320 threads, the digit rows were written by matmul_q_pieces_kernel
// and the copy engine brings each stage's part of them with the weights.
template <bool TRACE, bool XF32, bool PRE>
__global__ void __launch_bounds__(PRE ? 32u * (2u + MQ_SCALE_WARPS) : MQ_THREADS, 1)
matmul_q_fp4_kernel(const __grid_constant__ CUtensorMap tmap_wq, const __grid_constant__ CUtensorMap tmap_ws,
                    const __grid_constant__ CUtensorMap next_wq, const __grid_constant__ CUtensorMap next_ws,
                    const __grid_constant__ CUtensorMap tmap_b, MatmulQArgs a) {
    constexpr uint32_t NTHREADS = PRE ? 32u * (2u + MQ_SCALE_WARPS) : MQ_THREADS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);

    const uint32_t S = a.stages;
    const uint32_t MQ_STAGE_BYTES = matmul_q_stage_bytes(a.m);
    auto codes_of = [&](uint32_t s) { return base + s * MQ_STAGE_BYTES; };
    auto b_of = [&](uint32_t s) { return codes_of(s) + MQ_CODE_BYTES; };
    auto sfa_of = [&](uint32_t s) { return b_of(s) + matmul_q_b_bytes(a.m); };
    auto sfb_of = [&](uint32_t s) { return sfa_of(s) + MQ_SF_BYTES; };
    const uint32_t ws_base = base + S * MQ_STAGE_BYTES;                   // MQ_WS_SLOTS slots of scale bytes as stored
    const uint32_t bars = ws_base + MQ_WS_SLOTS * MQ_WS_SLOT_BYTES;
    auto raw_full = [&](uint32_t s) { return bars + 8u * s; };            // TMA bytes of the stage landed
    auto prep_full = [&](uint32_t s) { return bars + 8u * (S + s); };     // pieces and scale blocks written
    auto empty = [&](uint32_t s) { return bars + 8u * (2u * S + s); };    // the stage's MMAs are done
    const uint32_t acc_full = bars + 8u * 3u * S;
    auto ws_full = [&](uint32_t r) { return bars + 8u * (3u * S + 1u + r); };
    auto ws_empty = [&](uint32_t r) { return bars + 8u * (3u * S + 1u + MQ_WS_SLOTS + r); };    // all eight scale warps
    uint32_t* const misc = reinterpret_cast<uint32_t*>(smem + (bars - base) + (3u * S + 1u + 2u * MQ_WS_SLOTS) * 8u);
    uint32_t* const tmem_slot = misc;
    volatile uint32_t* const abort_flag = misc + 1;
    uint32_t* const tok_amax = misc + 2;                                   // [MQ_MAX_TOKENS]
    volatile uint32_t* const fix_flag = misc + 2 + MQ_MAX_TOKENS;
    volatile uint8_t* const nan_rows = reinterpret_cast<volatile uint8_t*>(misc + 48);   // [MQ_ROWS]: a NaN scale byte seen

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t split = blockIdx.x % a.k_splits, tile = blockIdx.x / a.k_splits;
    const uint32_t n0 = tile * MQ_ROWS;
    const uint32_t kb_all = a.k / MQ_STAGE_K;
    const uint32_t kb0 = split * a.kb_per_split;
    const uint32_t KB = (kb_all - kb0 < a.kb_per_split) ? (kb_all - kb0) : a.kb_per_split;
    const uint32_t N = a.m * MQ_PIECES;
    const bool wide = N > 128u;                               // more than 16 tokens: one accumulator, two scale blocks of B per MMA
    const uint32_t sfb_bytes = matmul_q_sfb_bytes(a.m);
    const long long t_start = clock64();

    if (warp == 0) {
        // one barrier per lane: the whole set is ready after a few instructions
        if (lane == 0) {
            prefetch_tensormap(&tmap_wq);
            prefetch_tensormap(&tmap_ws);
            if (PRE) prefetch_tensormap(&tmap_b);
            *abort_flag = 0;
        }
        if (lane < MQ_MAX_TOKENS) tok_amax[lane] = 0;
        const uint32_t nbar = 3u * S + 1u + 2u * MQ_WS_SLOTS;
        for (uint32_t b = lane; b < nbar; b += 32u) {
            uint32_t count = 1;                                                  // raw_full, empty, acc_full, ws_full
            if (b >= S && b < 2u * S) count = MQ_SCALE_WARPS / 2u + (PRE ? 0u : a.m);   // prep_full: four scale warps, one piece warp per token
            if (b >= 3u * S + 1u + MQ_WS_SLOTS) count = MQ_SCALE_WARPS;          // ws_empty: every scale warp
            mbar_init(bars + 8u * b, count);
        }
        __syncwarp();
        long long ta = 0;
        if (TRACE) ta = clock64();
        fence_mbar_init();
        if (TRACE && a.trace && lane == 0)
            a.trace[16ull * blockIdx.x + 9] = ((unsigned long long)(uint32_t)(clock64() - t_start) << 32) | (uint32_t)(ta - t_start);
    }
    if (tid >= 64u && tid < 64u + MQ_ROWS) nan_rows[tid - 64u] = 0;
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), MQ_TMEM_COLS);
        tmem_relinquish();
    }
    if (warp != 0) allow_dependents();
    // Warp 0 has set up every barrier itself and needs nothing from the others: it announces that and
    // goes on to its loads, the other warps meet here (named barrier 2).
    uint32_t tmem_base = 0;
    if (warp == 0) {
        asm volatile("bar.arrive 2, %0;" ::"r"(NTHREADS) : "memory");
    } else {
        tc_fence_before_sync();
        asm volatile("bar.sync 2, %0;" ::"r"(NTHREADS) : "memory");
        tc_fence_after_sync();
        tmem_base = *tmem_slot;
    }
    // x, r and y belong to the stream's order; the weights may be declared constant, and the warp
    // that loads them then starts while the launch ahead of this one is still running.
    if (!((a.flags & 1u) && warp == 0)) grid_dependency_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            RingPos ps;
            // Until its rings are full this warp waits for nothing.  Before its first wait for a slot to
            // come free it joins the stream's order itself: the other warps cannot free anything before
            // the launch ahead has finished, and a bounded wait must not run against that launch's time.
            bool in_order = !(a.flags & 1u);
            const uint32_t b_bytes = PRE ? N * 128u : 0u;                  // the tokens' digit rows of a stage
            uint32_t b_issued = 0;                                         // PRE: stages whose digit rows have been requested
            for (uint32_t kb = 0; kb < KB; kb++, ps.advance(S)) {
                const uint32_t s = ps.s;
                if (!in_order && (kb >= S || kb / MQ_WS_GROUP + 1u >= MQ_WS_SLOTS)) {
                    grid_dependency_wait();
                    in_order = true;
                }
                if (!mbar_wait(empty(s), ps.ph ^ 1u, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                    *abort_flag = 1;
                    break;
                }
                if (TRACE && a.trace && kb == 0) a.trace[16ull * blockIdx.x + 13] = (unsigned long long)clock64();
                if ((kb & (MQ_WS_GROUP - 1u)) == 0u) {
                    // Scale bytes, one group of four stages AHEAD of the codes (both groups at the start):
                    // re-laying them does not need the codes, so the scale warps work ahead of the copy
                    // engine's stream instead of starting when a stage lands.
                    const uint32_t g_first = kb == 0u ? 0u : kb / MQ_WS_GROUP + 1u, g_last = kb / MQ_WS_GROUP + 1u;
                    bool gave_up = false;
                    for (uint32_t wsi = g_first; wsi <= g_last && wsi * MQ_WS_GROUP < KB; wsi++) {
                        const uint32_t r = wsi % MQ_WS_SLOTS, wph = (wsi / MQ_WS_SLOTS) & 1u;
                        if (!mbar_wait(ws_empty(r), wph ^ 1u, abort_flag)) {
                            gave_up = true;
                            break;
                        }
                        mbar_arrive_expect_tx(ws_full(r), a.ws_pitch * MQ_ROWS);
                        tma_load_2d(ws_base + r * MQ_WS_SLOT_BYTES, &tmap_ws, (int)((kb0 + wsi * MQ_WS_GROUP) * (MQ_STAGE_K / 16)), (int)n0,
                                    ws_full(r));
                    }
                    if (gave_up) {
                        atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                        *abort_flag = 1;
                        break;
                    }
                }
                mbar_arrive_expect_tx(raw_full(s), MQ_CODE_BYTES + (PRE ? b_bytes + sfb_bytes : 0u));
                tma_load_2d(codes_of(s), &tmap_wq, (int)((kb0 + kb) * (MQ_STAGE_K / 2)), (int)n0, raw_full(s));
                if (kb + 1u == S || kb + 1u == KB) allow_dependents();       // the ring is filled (once is enough; twice is harmless)
                if (PRE) {
                    // The digit rows are written by the launch ahead (the pieces kernel): the first ring of
                    // weights goes out before that launch is waited for, the digit rows of those stages after.
                    if (!in_order && (kb + 1u == S || kb + 1u == KB)) {
                        grid_dependency_wait();
                        in_order = true;
                    }
                    if (in_order) {
                        for (; b_issued <= kb; b_issued++) {             // stages < S sit in slot = stage
                            const uint32_t sj = b_issued % S;
                            tma_load_2d(b_of(sj), &tmap_b, (int)((kb0 + b_issued) * (MQ_STAGE_K / 2)), 0, raw_full(sj));
                            tma_load_1d(sfb_of(sj), a.pre_sfb + (size_t)(kb0 + b_issued) * sfb_bytes, sfb_bytes, raw_full(sj));
                        }
                    }
                }
            }
            if (*abort_flag) {
                // copies still in flight land in this block's shared memory: give them a bounded time
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) {
                }
            } else {
                // what the next launch's blocks will ask for first, into L2 (block c for block c; the
                // blocks beyond this launch's grid are shared out in turns)
                for (uint32_t c = blockIdx.x; c < a.next_grid; c += gridDim.x) {
                    const uint32_t nsplit = c % a.next_k_splits, ntile = c / a.next_k_splits;
                    const uint32_t nkb0 = nsplit * a.next_kb_per_split;
                    uint32_t nkb = a.next_kb_all - nkb0 < a.next_kb_per_split ? a.next_kb_all - nkb0 : a.next_kb_per_split;
                    if (nkb > a.next_stages) nkb = a.next_stages;
                    for (uint32_t kb = 0; kb < nkb; kb++) {
                        if ((kb & (MQ_WS_GROUP - 1u)) == 0u)
                            tma_prefetch_l2_2d(&next_ws, (int)((nkb0 + kb) * (MQ_STAGE_K / 16)), (int)(ntile * MQ_ROWS));
                        tma_prefetch_l2_2d(&next_wq, (int)((nkb0 + kb) * (MQ_STAGE_K / 2)), (int)(ntile * MQ_ROWS));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- scale copies + MMA issue
        const uint32_t idesc = umma_idesc_mxf4nvf4(128u, N);
        if (TRACE && a.trace && lane == 0) a.trace[16ull * blockIdx.x + 15] = (unsigned long long)clock64();
        bool ok = true;
        long long w_raw = 0, w_prep = 0, t_issue = 0, t_first = 0;
        RingPos ps;
        for (uint32_t kb = 0; kb < KB; kb++, ps.advance(S)) {
            const uint32_t s = ps.s, ph = ps.ph;
            long long c0 = 0, c1 = 0, c2 = 0;
            if (TRACE) c0 = clock64();
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(raw_full(s), ph, abort_flag))) {
                atomicOr(a.status, ST_WAIT_X_FULL);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (TRACE) c1 = clock64();
            if (TRACE && a.trace && kb == 0 && lane == 0) a.trace[16ull * blockIdx.x + 14] = (unsigned long long)c1;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(prep_full(s), ph, abort_flag))) {
                atomicOr(a.status, ST_WAIT_W_FULL);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (TRACE) {
                c2 = clock64();
                w_raw += c1 - c0;
                w_prep += c2 - c1;
                if (kb == 0) t_first = c2;
            }
            tc_fence_after_sync();
            const uint32_t a_lo = umma_desc_lo(codes_of(s)), b_lo = umma_desc_lo(b_of(s));
            const uint32_t sfa_t = tmem_base + MQ_TMEM_SFA + 16u * s;
            const uint32_t sfb_t = tmem_base + (wide ? MQ_TMEM_SFB_WIDE + 32u * s : MQ_TMEM_SFB + 16u * s);
            const uint32_t sfb_cols = wide ? 8u : 4u, sfb_block = wide ? 1024u : 512u;     // per MMA
            const uint32_t d = tmem_base + ((!wide && (kb & 1u)) ? MQ_TMEM_D1 : 0u);       // two accumulators, alternating, when they fit
            if (elect_one()) {
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) {
                    tmem_cp_32x128b_warpx4(sfa_t + 4u * j, umma_desc_scale_block(sfa_of(s) + 512u * j));
                    tmem_cp_32x128b_warpx4(sfb_t + sfb_cols * j, umma_desc_scale_block(sfb_of(s) + sfb_block * j));
                    if (wide)          // rows 128-255 of B: the next four columns
                        tmem_cp_32x128b_warpx4(sfb_t + sfb_cols * j + 4u, umma_desc_scale_block(sfb_of(s) + sfb_block * j + 512u));
                }
                const uint32_t fresh = wide ? 1u : 2u;       // stages that start an accumulator
#pragma unroll
                for (uint32_t j = 0; j < 4; j++)
                    umma1_mxf4nvf4(d, a_lo + 2u * j, b_lo + 2u * j, idesc, sfa_t + 4u * j, sfb_t + sfb_cols * j,
                                   (kb >= fresh || j > 0u) ? 1u : 0u);
                umma_commit(empty(s));
            }
            __syncwarp();
            if (TRACE) t_issue += clock64() - c2;
        }
        if (ok && elect_one()) umma_commit(acc_full);
        __syncwarp();
        if (TRACE && a.trace && lane == 0) {
            unsigned long long* tr = a.trace + 16ull * blockIdx.x;
            tr[0] = (unsigned long long)t_start;
            tr[1] = (unsigned long long)t_first;     // first stage ready
            tr[2] = (unsigned long long)clock64();   // all MMAs issued
            tr[3] = (unsigned long long)w_raw;       // MMA warp: waiting for the copy engine
            tr[4] = (unsigned long long)w_prep;      // ... for the prep warps
            tr[5] = (unsigned long long)t_issue;     // ... issuing copies and MMAs
        }
    } else if (!PRE && warp >= 2u + MQ_SCALE_WARPS) {
        // ---------------------------------------------------------------- piece warps: x -> E2M1 digit rows
        const uint32_t xw = warp - (2u + MQ_SCALE_WARPS);
        const uint32_t xt = tid - 32u * (2u + MQ_SCALE_WARPS);
        const uint32_t items = KB * a.m;                      // item = (stage kb, token t), kb-major
        // A warp takes every PW-th item.  Its consecutive items must be at most S stages apart: a wait
        // on a stage's barrier can only tell "this turn of the ring" from the one before it.
        const uint32_t PW = (S * a.m < MQ_PIECE_WARPS) ? S * a.m : MQ_PIECE_WARPS;
        // one item's values for this lane: 8 consecutive values of K, as 8 halves or 8 floats
        struct Chunk {
            uint4 lo, hi;     // f16: lo only
        };
        auto load_chunk = [&](uint32_t kb, uint32_t t) {
            Chunk c;
            c.hi = make_uint4(0, 0, 0, 0);
            if (XF32) {
                const uint4* p4 = reinterpret_cast<const uint4*>(static_cast<const float*>(a.x) + (size_t)t * a.k) +
                                  (size_t)(kb0 + kb) * (MQ_STAGE_K / 4u) + 2u * lane;
                c.lo = __ldg(p4);
                c.hi = __ldg(p4 + 1);
            } else {
                c.lo = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(a.x) + (size_t)t * a.k) +
                             (size_t)(kb0 + kb) * (MQ_STAGE_K / 8u) + lane);
            }
            return c;
        };
        // the first item's values are on their way while the token maxima are found
        Chunk xv;
        xv.lo = xv.hi = make_uint4(0, 0, 0, 0);
        if (xw < PW && xw < items) xv = load_chunk(xw / a.m, xw % a.m);
        // largest magnitude of each token as f32 bits (its exponent gives the scale offset G); the
        // tokens' loads go out together
        for (uint32_t t0 = 0; t0 < a.m; t0 += 4u) {               // four tokens at a time (registers)
            uint32_t mx[4] = {0, 0, 0, 0};
            const uint4* xr = reinterpret_cast<const uint4*>(a.x);
            const uint32_t row_chunks = XF32 ? a.k / 4u : a.k / 8u;
#pragma unroll 4
            for (uint32_t i = xt; i < row_chunks; i += 32u * MQ_PIECE_WARPS) {
                uint4 v[4];
#pragma unroll
                for (uint32_t t = 0; t < 4; t++)
                    v[t] = t0 + t < a.m ? __ldg(xr + (size_t)(t0 + t) * row_chunks + i) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (uint32_t t = 0; t < 4; t++) {
                    if (XF32) {
                        mx[t] = max(max(mx[t], v[t].x & 0x7FFFFFFFu), v[t].y & 0x7FFFFFFFu);
                        mx[t] = max(max(mx[t], v[t].z & 0x7FFFFFFFu), v[t].w & 0x7FFFFFFFu);
                    } else {
                        mx[t] = __vmaxu2(mx[t], v[t].x & 0x7FFF7FFFu);
                        mx[t] = __vmaxu2(mx[t], v[t].y & 0x7FFF7FFFu);
                        mx[t] = __vmaxu2(mx[t], v[t].z & 0x7FFF7FFFu);
                        mx[t] = __vmaxu2(mx[t], v[t].w & 0x7FFF7FFFu);
                    }
                }
            }
#pragma unroll
            for (uint32_t t = 0; t < 4; t++) {
                if (t0 + t < a.m) {
                    uint32_t r = mx[t];
                    if (!XF32) {
                        r = max(r & 0xFFFFu, r >> 16);
                        r = __float_as_uint(__half2float(__ushort_as_half((unsigned short)r)));   // exact; inf and NaN stay so
                    }
                    r = __reduce_max_sync(0xFFFFFFFFu, r);
                    if (lane == 0) atomicMax(tok_amax + t0 + t, r);
                }
            }
        }
        // B's scale blocks start as zeros: rows nobody writes must not hold stray NaN patterns
        for (uint32_t i = xt; i < S * (sfb_bytes / 16u); i += 32u * MQ_PIECE_WARPS) {
            const uint32_t s = i / (sfb_bytes / 16u), o = i % (sfb_bytes / 16u);
            *reinterpret_cast<uint4*>(smem + (sfb_of(s) - base) + 16u * o) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("bar.sync 1, %0;" ::"r"(32u * MQ_PIECE_WARPS) : "memory");
        long long p_empty = 0, p_t0 = 0;
        if (TRACE) p_t0 = clock64();
        for (uint32_t it = (xw < PW ? xw : items); it < items; it += PW) {
            const uint32_t kb = it / a.m, tok = it - kb * a.m;
            const uint32_t s = kb % S, ph = (kb / S) & 1u;
            const Chunk xc = xv;
            if (it + PW < items) xv = load_chunk((it + PW) / a.m, (it + PW) % a.m);
            const uint32_t te8 = tok_amax[tok] >> 23;                 // the token's largest f32 exponent field
            // ---- 8 values of the token: K offsets 8 lane .. 8 lane + 7 of the stage
            uint32_t fb[8], w[8], e8;
            mq_widen<XF32>(xc.lo, xc.hi, fb);
            mq_digits(fb, w, e8);
            long long q0c = 0;
            if (TRACE) q0c = clock64();
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty(s), ph ^ 1u, abort_flag))) {
                atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                *abort_flag = 1;
                break;
            }
            if (TRACE) p_empty += clock64() - q0c;
            uint8_t* const bt = smem + (b_of(s) - base) + (tok * MQ_PIECES) * 128u + 4u * (lane & 3u);
#pragma unroll
            for (uint32_t pc = 0; pc < MQ_PIECES; pc++)      // row 8 tok + pc: its chunk XOR is pc
                *reinterpret_cast<uint32_t*>(bt + pc * 128u + (((lane >> 2) ^ pc) << 4)) = w[pc];
            // scales of this group's pieces: 2^(8 - (token max - group max) - 2 piece)
            const int q0 = 8 - (int)(te8 - e8);
            const uint32_t grp = lane >> 1;                  // group of 16 within the stage
            // row n = 8 tok + piece of the block: 16 bytes per (n % 32), 4 bytes per (n / 32), one per group
            uint8_t* const sb = smem + (sfb_of(s) - base);
#pragma unroll
            for (uint32_t i = 0; i < 4; i++) {
                const uint32_t pc = 4u * (lane & 1u) + i;
                sb[mq_sfb_offset(tok * MQ_PIECES + pc, grp, wide)] = (uint8_t)mq_ue4m3_pow2(q0 - 2 * (int)pc);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(prep_full(s));
        }
        if (TRACE && a.trace && xt == 0) {
            unsigned long long* tr = a.trace + 16ull * blockIdx.x + 11;
            tr[0] = (unsigned long long)(clock64() - p_t0);   // piece loop of warp 0, total
            tr[1] = (unsigned long long)p_empty;              // ... waiting for a free stage
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- scale warps (2-5 also run the epilogue)
        // Two sets of four warps take the even and the odd stages: one warp's pass over a stage is a
        // short chain of dependent instructions that a single warp cannot overlap with itself.
        const uint32_t set = (warp - 2u) >> 2;
        const uint32_t row = 32u * (warp & 3u) + lane;        // the lanes of tensor memory this warp may read
        const float g = __ldg(a.wg + n0 + row);
        bool ok = true;
        long long p_empty = 0, p_raw = 0, p_t0 = 0;
        if (TRACE) p_t0 = clock64();
        RingPos ps;
        if (set) ps.advance(S);
        for (uint32_t kb = set; kb < KB; kb += 2u, ps.advance(S), ps.advance(S)) {
            const uint32_t s = ps.s, ph = ps.ph;
            long long q0c = 0, q1c = 0;
            if (TRACE) q0c = clock64();
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty(s), ph ^ 1u, abort_flag))) {
                atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (TRACE) q1c = clock64();
            // ---- this row's 16 scale bytes of the stage -> four scale blocks
            const uint32_t wsi = kb / MQ_WS_GROUP, wr = wsi % MQ_WS_SLOTS, wph = (wsi / MQ_WS_SLOTS) & 1u;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(ws_full(wr), wph, abort_flag))) {
                atomicOr(a.status, ST_WAIT_X_FULL);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (TRACE) {
                p_empty += q1c - q0c;
                p_raw += clock64() - q1c;
            }
            const uint4 sc = *reinterpret_cast<const uint4*>(smem + (ws_base - base) + wr * MQ_WS_SLOT_BYTES + row * a.ws_pitch +
                                                             16u * (kb & (MQ_WS_GROUP - 1u)));
            if ((kb & (MQ_WS_GROUP - 1u)) >= MQ_WS_GROUP - 2u || kb + 2u >= KB) {   // this warp's last stage of the group
                __syncwarp();
                if (lane == 0) mbar_arrive(ws_empty(wr));
            }
            uint32_t sv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) {
                uint32_t v = sv[j];
                if (v & 0x80808080u) {
                    // negative scales: move the sign into the 16 codes of the group (once they are here)
                    if (!mbar_wait(raw_full(s), ph, abort_flag)) {
                        atomicOr(a.status, ST_WAIT_X_FULL);
                        *abort_flag = 1;
                    }
                    for (uint32_t i = 0; i < 4; i++) {
                        if ((v >> (8u * i + 7u)) & 1u) {
                            const uint32_t bi = 4u * j + i;
                            uint32_t* cw = reinterpret_cast<uint32_t*>(smem + (codes_of(s) - base) + row * 128u +
                                                                       (((bi >> 1) ^ (row & 7u)) << 4) + 8u * (bi & 1u));
                            cw[0] ^= 0x88888888u;
                            cw[1] ^= 0x88888888u;
                        }
                    }
                    v &= 0x7F7F7F7Fu;
                }
                const uint32_t z = v ^ 0x7F7F7F7Fu;
                if ((z - 0x01010101u) & ~z & 0x80808080u) {      // some byte may be 0x7f: look at each
                    for (uint32_t i = 0; i < 4; i++) {
                        if (((v >> (8u * i)) & 0xFFu) == 0x7Fu) {
                            nan_rows[row] = 1;
                            v &= ~(0xFFu << (8u * i));
                        }
                    }
                }
                *reinterpret_cast<uint32_t*>(smem + (sfa_of(s) - base) + 512u * j + (row & 31u) * 16u + (row >> 5) * 4u) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(prep_full(s));
        }
        if (TRACE && a.trace && tid == 64) {
            unsigned long long* tr = a.trace + 16ull * blockIdx.x + 6;
            tr[0] = (unsigned long long)(clock64() - p_t0);   // scale loop of warp 2, total
            tr[1] = (unsigned long long)p_empty;              // ... waiting for a free stage
            tr[2] = (unsigned long long)p_raw;                // ... waiting for the scale bytes
        }
        // ---------------------------------------------------------------- epilogue (warps 2-5)
        if (set == 0u) {
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
            const bool row_nan = nan_rows[row] != 0;
            const uint32_t lane_base = tmem_base + ((32u * (warp & 3u)) << 16);
            const bool to_partial = a.k_splits > 1u;
            const bool two_acc = !wide && KB > 1u;
            float* const out = to_partial ? a.partial + (size_t)split * a.m * a.n : a.y;
            for (uint32_t t = 0; t < a.m; t++) {
                uint32_t d0[8], d1[8];
                tmem_ld_32x32b_x8(lane_base + 8u * t, d0);
                if (two_acc) tmem_ld_32x32b_x8(lane_base + MQ_TMEM_D1 + 8u * t, d1);
                tmem_ld_wait();
                float v = 0.0f;
#pragma unroll
                for (int pc = 7; pc >= 0; pc--) {                // small pieces first
                    float c = __uint_as_float(d0[pc]);
                    if (two_acc) c += __uint_as_float(d1[pc]);
                    v += c;
                }
                const uint32_t te = (PRE ? __ldg(a.pre_amax + t) : tok_amax[t]) >> 23;
                const float tscale = te >= 16u ? __uint_as_float((te - 8u) << 23) : 0.0f;   // 2^G, G = E_token - 8
                v = v * tscale * g;
                if (row_nan || te == 255u) v = __uint_as_float(0x7FC00000u);
                const size_t o = (size_t)t * a.n + n0 + row;
                if (!to_partial && a.r) v += __ldg(a.r + o);
                out[o] = v;
            }
        }
        if (a.k_splits > 1u) {
            // The last block of a row tile to get here adds up the splits, always in the order of the
            // splits, so the result does not depend on which block that is.  (A block that gave up
            // above still counts itself: the counter must be back at zero for the next launch.)
            __threadfence();
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (warp == 2u && lane == 0) *fix_flag = atomicAdd(a.counters + tile, 1u);
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (*fix_flag == a.k_splits - 1u) {
                __threadfence();
                for (uint32_t t = 0; t < a.m; t++) {
                    const size_t o = (size_t)t * a.n + n0 + row;
                    float sum = 0.0f;
                    for (uint32_t sp = 0; sp < a.k_splits; sp++) sum += __ldcg(a.partial + (size_t)sp * a.m * a.n + o);
                    if (a.r) sum += __ldg(a.r + o);
                    a.y[o] = sum;
                }
                if (warp == 2u && lane == 0) a.counters[tile] = 0;
            }
        }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (TRACE && a.trace && tid == 0) a.trace[16ull * blockIdx.x + 10] = (unsigned long long)clock64();   // block done
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, MQ_TMEM_COLS);
    }
}

// The tokens' digit rows, once per launch, for the PRE variant of the kernel above: blocks (t, *) take token t,
// each finds the token's largest magnitude itself and takes every gridDim.y-th set of 32 stages.
//   pieces [8 m][k / 2] bytes: row 8 t + p holds piece p of token t, packed like wq (a tensor map with the
//                              128-byte swizzle brings 8 m x 128 bytes of it per stage);
//   sfb    [k / 256][2048 or 4096] bytes: per stage the scale blocks of B (rows past 8 m stay zero);
//   amax   [m]: the token's largest magnitude as f32 bits.
// It follows the previous launch of the same pipeline in the stream, which may still be reading these
// buffers: nothing is written before grid_dependency_wait().
// XMODE: 0 = f16 activations, 1 = f32, 2 = int16 activations with one f32 scale per 16 values (`xs`), as
// lex_msl::int8::quant16 leaves them (crates/lex-msl/src/int8.rs:47-114): the value is q * xs in f32.
template <int XMODE>
__global__ void __launch_bounds__(1024, 1)
matmul_q_pieces_kernel(const void* __restrict__ x, uint32_t k, uint8_t* __restrict__ pieces, uint8_t* __restrict__ sfb,
                       uint32_t* __restrict__ amax, const float* __restrict__ xs) {
    constexpr bool XF32 = XMODE == 1, Q16 = XMODE == 2;
    const bool wide = gridDim.x > 16u;                        // tokens = gridDim.x
    const uint32_t sfb_stage = matmul_q_sfb_bytes(gridDim.x);
    __shared__ uint32_t s_amax;
    const uint32_t tok = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid == 0) s_amax = 0;
    allow_dependents();
    grid_dependency_wait();
    __syncthreads();
    const uint4* xr = XF32 ? reinterpret_cast<const uint4*>(static_cast<const float*>(x) + (size_t)tok * k)
                           : reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + (size_t)tok * k);
    const float* xsr = Q16 ? xs + (size_t)tok * (k / 16u) : nullptr;
    // eight int16 (one 16-byte load) times their group's scale, as f32 bit patterns
    auto q16_widen = [](const uint4& v, float sc, uint32_t (&fb)[8]) {
        const uint32_t hw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            fb[2 * i] = __float_as_uint(__fmul_rn((float)(short)(hw[i] & 0xFFFFu), sc));
            fb[2 * i + 1] = __float_as_uint(__fmul_rn((float)(short)(hw[i] >> 16), sc));
        }
    };
    const uint32_t row_chunks = XF32 ? k / 4u : k / 8u;
    uint32_t mx = 0;
#pragma unroll 4
    for (uint32_t i = tid; i < row_chunks; i += 1024u) {
        const uint4 v = __ldg(xr + i);
        if (XF32) {
            mx = max(max(mx, v.x & 0x7FFFFFFFu), v.y & 0x7FFFFFFFu);
            mx = max(max(mx, v.z & 0x7FFFFFFFu), v.w & 0x7FFFFFFFu);
        } else if (Q16) {
            uint32_t fb[8];
            q16_widen(v, __ldg(xsr + (i >> 1)), fb);
#pragma unroll
            for (uint32_t j = 0; j < 8; j++) mx = max(mx, fb[j] & 0x7FFFFFFFu);
        } else {
            mx = __vmaxu2(mx, v.x & 0x7FFF7FFFu);
            mx = __vmaxu2(mx, v.y & 0x7FFF7FFFu);
            mx = __vmaxu2(mx, v.z & 0x7FFF7FFFu);
            mx = __vmaxu2(mx, v.w & 0x7FFF7FFFu);
        }
    }
    if (!XF32 && !Q16) {
        mx = max(mx & 0xFFFFu, mx >> 16);
        mx = __float_as_uint(__half2float(__ushort_as_half((unsigned short)mx)));
    }
    mx = __reduce_max_sync(0xFFFFFFFFu, mx);
    if (lane == 0) atomicMax(&s_amax, mx);
    __syncthreads();
    const uint32_t tmax = s_amax, te8 = tmax >> 23;
    if (tid == 0 && blockIdx.y == 0) amax[tok] = tmax;
    for (uint32_t kb = blockIdx.y * 32u + warp; kb < k / MQ_STAGE_K; kb += 32u * gridDim.y) {
        uint4 lo, hi = make_uint4(0, 0, 0, 0);
        if (XF32) {
            lo = __ldg(xr + (size_t)kb * (MQ_STAGE_K / 4u) + 2u * lane);
            hi = __ldg(xr + (size_t)kb * (MQ_STAGE_K / 4u) + 2u * lane + 1u);
        } else {
            lo = __ldg(xr + (size_t)kb * (MQ_STAGE_K / 8u) + lane);
        }
        uint32_t fb[8], w[8], e8;
        if (Q16) q16_widen(lo, __ldg(xsr + (size_t)kb * (MQ_STAGE_K / 16u) + (lane >> 1)), fb);
        else mq_widen<XF32>(lo, hi, fb);
        mq_digits(fb, w, e8);
        const int q0 = 8 - (int)(te8 - e8);
        const uint32_t grp = lane >> 1;
        uint8_t sv[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) sv[i] = (uint8_t)mq_ue4m3_pow2(q0 - 2 * (int)(4u * (lane & 1u) + i));
#pragma unroll
        for (uint32_t pc = 0; pc < MQ_PIECES; pc++)
            *reinterpret_cast<uint32_t*>(pieces + (size_t)(tok * MQ_PIECES + pc) * (k / 2u) + kb * 128u + 4u * lane) = w[pc];
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            const uint32_t pc = 4u * (lane & 1u) + i;
            sfb[(size_t)kb * sfb_stage + mq_sfb_offset(tok * MQ_PIECES + pc, grp, wide)] = sv[i];
        }
    }
}

}  // namespace lexb
