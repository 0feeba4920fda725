// A run of matmul_q steps of one step list (same t <= 8 and k; see matmul_q_fp4_sm100.cuh) as ONE persistent
// kernel.  The runtime issues a layer's dispatches as a list (`Gpu::run_launches`,
// crates/lex-cuda/src/device.rs:650-672); consecutive steps of it often read the same activations against
// different weights (gate and up of one MLP, the q/k/v projections).
//
// A kernel that allocates tensor memory gets an SM to itself, so separate launches cannot overlap on an SM:
// every launch pays its set-up, the first bytes' trip from DRAM and its tail with the memory system idle.
// Here the run's row tiles (128 rows of one step, all of K) are numbered through the steps and block b takes
// tiles b, b + grid, b + 2 grid, ...: every SM has work whatever the steps' tile counts are (136 tiles of
// n = 17408 leave 12 of 148 SMs idle in a launch of their own, 224 tiles of n = 28672 need two waves), and a
// block's rings never drain: the copy engine is into the next tile's weights while this tile's last stages
// are multiplied and stored.  Nothing orders the tiles of different blocks, so the host only puts a step into a
// run if nothing it reads (x, r) is written, and nothing it writes (y) read or written, by a step already in the
// run (it compares the buffers' address ranges); a step that does depend on the run starts a new launch, and
// the stream orders it as usual.  (A version that waited inside the kernel - every block counts itself in after
// storing a step, the next step's x is read once the count is complete - was measured: 14.3 us per step
// against 12.2 us for separate launches, because nothing can be prefetched past the wait but one ring.)
// Blocks never wait for one another.  The weights are declared constant by every step of a run, so the copy
// engine's warp starts on them while the launch ahead is still running (programmatic stream serialization) and
// joins the stream's order before its first wait for a slot; every other warp joins it before touching x, r or y.
// The job table is never rewritten once it has been copied to the device, so it may be read before that.
//
// Roles: warp 0 copy engine, warp 1 scale copies + MMAs, warps 2-5 / 6-9 scale re-lay of even / odd stages,
// warps 10-13 epilogue, and - PRE = false, 576 threads - warps 14-17 the tokens' digit rows.  Every block derives
// the same digit rows, which bounds the kernel from 3 tokens on; PRE = true (448 threads) has them derived once
// per run and activation buffer by matmul_q_pieces_kernel, launched ahead, and the copy engine brings each
// stage's digit rows and scale blocks with the weights (nothing of a run writes its activations).  Two sets of
// accumulators (by the parity of the block's tile count) let a tile's MMAs start while the tile before is being
// stored.
#pragma once
#include "matmul_q_fp4_sm100.cuh"

namespace lexb {

struct alignas(64) MqChainJob {
    CUtensorMap wq, ws;      // this step's packed codes and scale bytes
    const void* x;           // [m, k]
    const float* wg;         // [n]
    const float* r;          // [m, n] or null
    float* y;                // [m, n]
    uint32_t n;              // rows of this step's weights
    uint32_t tile_end;       // the run's tile count up to and including this step
    // PRE: what matmul_q_pieces_kernel wrote for this step's x
    const uint8_t* pre_sfb;  // [k / 256][2048] scale blocks of the digit rows
    const uint32_t* pre_amax;// [m] largest magnitudes, f32 bits
    CUtensorMap pre;         // digit rows [8 m][k / 2]
    uint64_t pad[1];
};
static_assert(sizeof(MqChainJob) % 64 == 0, "tensor maps of a job table sit on 64-byte boundaries");

struct MqChainArgs {
    const MqChainJob* jobs;
    uint32_t n_jobs, n_tiles;
    uint32_t tiles_per_job;  // every step has this many row tiles, or 0: they differ and the table is walked
    uint32_t m, k, stages, ws_pitch;
    uint32_t* status;
};

constexpr uint32_t MQC_PIECE_WARPS = 4;
constexpr uint32_t MQC_WARP_EPI = 2u + MQ_SCALE_WARPS;                 // 10
constexpr uint32_t MQC_WARP_PIECE = MQC_WARP_EPI + 4u;                 // 14
constexpr uint32_t MQC_THREADS = 32u * (MQC_WARP_PIECE + MQC_PIECE_WARPS);
// Tensor memory: two sets of two accumulators of 32 columns (up to 4 tokens) or 64 (up to 8), then the scale
// blocks of A and of B, 16 columns per stage each: 128 + 256 or 256 + 256 of the 512 columns.
__host__ __device__ constexpr uint32_t matmul_q_chain_acc_cols(uint32_t m) { return m <= 4u ? 32u : 64u; }
constexpr uint32_t MQC_MAX_TOKENS = 8;

__host__ __device__ constexpr uint32_t matmul_q_chain_smem_bytes(uint32_t stages, uint32_t m) {
    return stages * matmul_q_stage_bytes(m <= 4u ? 4u : 8u) + MQ_WS_SLOTS * MQ_WS_SLOT_BYTES + (3u * stages + 4u + 2u * MQ_WS_SLOTS) * 8u + 64u +
           2u * MQ_ROWS + 1024u;
}

constexpr uint32_t MQC_THREADS_PRE = 32u * MQC_WARP_PIECE;

template <bool XF32, bool PRE>
__global__ void __launch_bounds__(PRE ? MQC_THREADS_PRE : MQC_THREADS, 1) matmul_q_chain_kernel(MqChainArgs a) {
    constexpr uint32_t NTHREADS = PRE ? MQC_THREADS_PRE : MQC_THREADS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);

    const uint32_t S = a.stages;
    const uint32_t MB = a.m <= 4u ? 4u : 8u;                               // the token count the stages are sized for
    const uint32_t STAGE_BYTES = matmul_q_stage_bytes(MB);
    const uint32_t ACC = matmul_q_chain_acc_cols(a.m), TMEM_SET = 2u * ACC;
    const uint32_t TMEM_SFA = 2u * TMEM_SET, TMEM_SFB = TMEM_SFA + 16u * MQ_MAX_STAGES;
    auto codes_of = [&](uint32_t s) { return base + s * STAGE_BYTES; };
    auto b_of = [&](uint32_t s) { return codes_of(s) + MQ_CODE_BYTES; };
    auto sfa_of = [&](uint32_t s) { return b_of(s) + matmul_q_b_bytes(MB); };
    auto sfb_of = [&](uint32_t s) { return sfa_of(s) + MQ_SF_BYTES; };
    const uint32_t ws_base = base + S * STAGE_BYTES;
    const uint32_t bars = ws_base + MQ_WS_SLOTS * MQ_WS_SLOT_BYTES;
    auto raw_full = [&](uint32_t s) { return bars + 8u * s; };
    auto prep_full = [&](uint32_t s) { return bars + 8u * (S + s); };
    auto empty = [&](uint32_t s) { return bars + 8u * (2u * S + s); };
    auto acc_full = [&](uint32_t set) { return bars + 8u * (3u * S + set); };            // a step's MMAs are done
    auto acc_empty = [&](uint32_t set) { return bars + 8u * (3u * S + 2u + set); };      // ... and stored: four epilogue warps
    auto ws_full = [&](uint32_t r) { return bars + 8u * (3u * S + 4u + r); };
    auto ws_empty = [&](uint32_t r) { return bars + 8u * (3u * S + 4u + MQ_WS_SLOTS + r); };
    const uint32_t nbar = 3u * S + 4u + 2u * MQ_WS_SLOTS;
    uint32_t* const misc = reinterpret_cast<uint32_t*>(smem + (bars - base) + nbar * 8u);
    uint32_t* const tmem_slot = misc;
    volatile uint32_t* const abort_flag = misc + 1;
    uint32_t* const tok_amax = misc + 2;                                  // [2 sets][4 tokens]
    volatile uint8_t* const nan_rows = reinterpret_cast<volatile uint8_t*>(misc + 16);    // [2 sets][MQ_ROWS]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t KB = a.k / MQ_STAGE_K;
    const uint32_t GP = (KB + MQ_WS_GROUP - 1u) / MQ_WS_GROUP;             // scale-byte groups per step
    const uint32_t N = a.m * MQ_PIECES;
    // this block's tiles: blockIdx.x + i * gridDim.x, i < T
    const uint32_t T = blockIdx.x < a.n_tiles ? (a.n_tiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
    // step and first row of the block's i-th tile; `j` is the caller's cursor into the steps (tiles ascend)
    auto locate = [&](uint32_t i, uint32_t& j) -> uint32_t {
        const uint32_t tile = blockIdx.x + i * gridDim.x;
        if (a.tiles_per_job) {       // (a walk is one trip to L2 per step passed: with few tiles per step that is most of a tile's time)
            j = tile / a.tiles_per_job;
            return (tile - j * a.tiles_per_job) * MQ_ROWS;
        }
        while (j + 1u < a.n_jobs && tile >= a.jobs[j].tile_end) j++;
        return (tile - (j ? a.jobs[j - 1u].tile_end : 0u)) * MQ_ROWS;
    };

    if (warp == 0) {
        if (lane == 0) *abort_flag = 0;
        if (lane < 8u) tok_amax[lane] = 0;
        for (uint32_t b = lane; b < nbar; b += 32u) {
            uint32_t count = 1;                                                       // raw_full, empty, acc_full, ws_full
            if (b >= S && b < 2u * S) count = MQ_SCALE_WARPS / 2u + (PRE ? 0u : a.m); // prep_full
            if (b >= 3u * S + 2u && b < 3u * S + 4u) count = 4u;                      // acc_empty: the epilogue warps
            if (b >= 3u * S + 4u + MQ_WS_SLOTS) count = MQ_SCALE_WARPS;               // ws_empty
            mbar_init(bars + 8u * b, count);
        }
        __syncwarp();
        fence_mbar_init();
    }
    for (uint32_t i = tid; i < 2u * MQ_ROWS; i += NTHREADS) nan_rows[i] = 0;
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), MQ_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (warp != 0) {
        allow_dependents();
        grid_dependency_wait();
    }

    if (warp == 0) {
        // ---------------------------------------------------------------- copy engine: every step's weights, in order
        if (lane == 0) {
            RingPos ps;
            uint32_t g_issued = 0;                    // scale-byte groups requested so far (flat over the block's tiles)
            const uint32_t TG = T * GP;
            uint32_t gj = 0, g_tile = ~0u, g_n0 = 0;  // the scale bytes' own cursor (they run ahead of the codes); the job
                                                      // table is read once per tile, not per group
            // Nothing is waited for until the rings are full.  Before its first real wait this warp joins the
            // stream's order: the warps that free the slots wait for the launch ahead, and a bounded wait must
            // not run against that launch's time.
            bool in_order = false;
            auto join_order = [&]() {
                if (!in_order) {
                    allow_dependents();
                    grid_dependency_wait();
                    in_order = true;
                }
            };
            auto issue_group = [&](uint32_t G) -> bool {
                const uint32_t r = G % MQ_WS_SLOTS, wph = (G / MQ_WS_SLOTS) & 1u;
                if (G >= MQ_WS_SLOTS) join_order();
                if (!mbar_wait(ws_empty(r), wph ^ 1u, abort_flag)) return false;
                const uint32_t i = G / GP, g = G - i * GP;
                if (i != g_tile) {
                    g_tile = i;
                    g_n0 = locate(i, gj);
                }
                const uint32_t gn0 = g_n0;
                mbar_arrive_expect_tx(ws_full(r), a.ws_pitch * MQ_ROWS);
                tma_load_2d(ws_base + r * MQ_WS_SLOT_BYTES, &a.jobs[gj].ws, (int)(g * MQ_WS_GROUP * (MQ_STAGE_K / 16)), (int)gn0, ws_full(r));
                return true;
            };
            bool ok = true;
            uint32_t j = 0, filled = 0;
            uint32_t b_issued = 0, bj = 0;            // PRE: stages whose digit rows have been requested, and their cursor
            const uint32_t b_bytes = PRE ? N * 128u : 0u;
            uint32_t b_tile = 0, b_kb = 0;
            const uint8_t* b_sfb = nullptr;
            if (PRE) {
                locate(0, bj);
                b_sfb = a.jobs[bj].pre_sfb;
            }
            for (uint32_t ti = 0; ti < T && ok; ti++) {
                const uint32_t n0 = locate(ti, j);
                for (uint32_t kb = 0; kb < KB; kb++, ps.advance(S), filled++) {
                    const uint32_t s = ps.s;
                    if (filled >= S) join_order();
                    if (!mbar_wait(empty(s), ps.ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    if ((kb & (MQ_WS_GROUP - 1u)) == 0u) {
                        // scale bytes one group ahead of the codes (two at the very start)
                        const uint32_t want = ti * GP + kb / MQ_WS_GROUP + 2u;
                        while (g_issued < want && g_issued < TG && ok) ok = issue_group(g_issued++);
                        if (!ok) break;
                    }
                    mbar_arrive_expect_tx(raw_full(s), MQ_CODE_BYTES + (PRE ? b_bytes + MQ_SF_BYTES : 0u));
                    tma_load_2d(codes_of(s), &a.jobs[j].wq, (int)(kb * (MQ_STAGE_K / 2)), (int)n0, raw_full(s));
                    if (PRE) {
                        // The digit rows are written by the launch ahead: the first ring of weights goes out
                        // before that launch is waited for, the digit rows of those stages (slot = stage) after.
                        if (filled + 1u == S || (ti + 1u == T && kb + 1u == KB)) join_order();
                        if (in_order) {
                            for (; b_issued <= filled; b_issued++, b_kb++) {
                                if (b_kb == KB) {            // the next tile of this block (the job table is not read per stage)
                                    b_kb = 0;
                                    locate(++b_tile, bj);
                                    b_sfb = a.jobs[bj].pre_sfb;
                                }
                                const uint32_t bs = b_issued % S;
                                tma_load_2d(b_of(bs), &a.jobs[bj].pre, (int)(b_kb * (MQ_STAGE_K / 2)), 0, raw_full(bs));
                                tma_load_1d(sfb_of(bs), b_sfb + (size_t)b_kb * MQ_SF_BYTES, MQ_SF_BYTES, raw_full(bs));
                            }
                        }
                    }
                }
            }
            join_order();
            if (!ok) {
                atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                *abort_flag = 1;
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) {
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- scale copies + MMA issue
        const uint32_t idesc = umma_idesc_mxf4nvf4(128u, N);
        bool ok = true;
        RingPos ps;
        for (uint32_t ti = 0; ti < T && ok; ti++) {
            const uint32_t set = ti & 1u, use = ti >> 1;
            // the accumulators of this set must have been stored (the block's tile before last)
            if (use > 0u && !__all_sync(0xFFFFFFFFu, mbar_wait(acc_empty(set), (use - 1u) & 1u, abort_flag))) {
                atomicOr(a.status, ST_WAIT_ACC);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after_sync();
            for (uint32_t kb = 0; kb < KB; kb++, ps.advance(S)) {
                const uint32_t s = ps.s, ph = ps.ph;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(raw_full(s), ph, abort_flag)) ||
                    !__all_sync(0xFFFFFFFFu, mbar_wait(prep_full(s), ph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_W_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_lo = umma_desc_lo(codes_of(s)), b_lo = umma_desc_lo(b_of(s));
                const uint32_t sfa_t = tmem_base + TMEM_SFA + 16u * s, sfb_t = tmem_base + TMEM_SFB + 16u * s;
                const uint32_t d = tmem_base + set * TMEM_SET + ((kb & 1u) ? ACC : 0u);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t q = 0; q < 4; q++) {
                        tmem_cp_32x128b_warpx4(sfa_t + 4u * q, umma_desc_scale_block(sfa_of(s) + 512u * q));
                        tmem_cp_32x128b_warpx4(sfb_t + 4u * q, umma_desc_scale_block(sfb_of(s) + 512u * q));
                    }
#pragma unroll
                    for (uint32_t q = 0; q < 4; q++)
                        umma1_mxf4nvf4(d, a_lo + 2u * q, b_lo + 2u * q, idesc, sfa_t + 4u * q, sfb_t + 4u * q,
                                       (kb >= 2u || q > 0u) ? 1u : 0u);
                    umma_commit(empty(s));
                    if (kb + 1u == KB) umma_commit(acc_full(set));
                }
                __syncwarp();
            }
        }
        __syncwarp();
    } else if (warp < MQC_WARP_EPI) {
        // ---------------------------------------------------------------- scale warps: even / odd stages of the whole list
        const uint32_t par = (warp - 2u) >> 2;
        const uint32_t row = 32u * (warp & 3u) + lane;
        bool ok = true;
        RingPos ps;
        uint32_t gs = 0;                                  // stage index over the block's tiles
        for (uint32_t ti = 0; ti < T && ok; ti++) {
            const uint32_t set = ti & 1u, use = ti >> 1;
            bool flags_free = use == 0u;                  // this set's NaN flags are cleared by the epilogue of the tile before last
            for (uint32_t kb = 0; kb < KB; kb++, ps.advance(S), gs++) {
                if ((gs & 1u) != par) continue;
                const uint32_t s = ps.s, ph = ps.ph;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty(s), ph ^ 1u, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t G = ti * GP + kb / MQ_WS_GROUP, wr = G % MQ_WS_SLOTS, wph = (G / MQ_WS_SLOTS) & 1u;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(ws_full(wr), wph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_X_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint4 sc = *reinterpret_cast<const uint4*>(smem + (ws_base - base) + wr * MQ_WS_SLOT_BYTES + row * a.ws_pitch +
                                                                 16u * (kb & (MQ_WS_GROUP - 1u)));
                // this warp's last stage of the group: the stages of a group alternate between the two sets
                // of warps by the parity of the list-wide stage index
                bool last_of_group = true;
                for (uint32_t q = kb + 1u; q < KB && (q / MQ_WS_GROUP) == (kb / MQ_WS_GROUP); q++)
                    if (((gs + (q - kb)) & 1u) == par) last_of_group = false;
                if (last_of_group) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ws_empty(wr));
                }
                uint32_t sv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (uint32_t q = 0; q < 4; q++) {
                    uint32_t v = sv[q];
                    if (v & 0x80808080u) {
                        if (!mbar_wait(raw_full(s), ph, abort_flag)) {
                            atomicOr(a.status, ST_WAIT_X_FULL);
                            *abort_flag = 1;
                        }
                        for (uint32_t i = 0; i < 4; i++) {
                            if ((v >> (8u * i + 7u)) & 1u) {
                                const uint32_t bi = 4u * q + i;
                                uint32_t* cw = reinterpret_cast<uint32_t*>(smem + (codes_of(s) - base) + row * 128u +
                                                                           (((bi >> 1) ^ (row & 7u)) << 4) + 8u * (bi & 1u));
                                cw[0] ^= 0x88888888u;
                                cw[1] ^= 0x88888888u;
                            }
                        }
                        v &= 0x7F7F7F7Fu;
                    }
                    const uint32_t z = v ^ 0x7F7F7F7Fu;
                    if ((z - 0x01010101u) & ~z & 0x80808080u) {
                        for (uint32_t i = 0; i < 4; i++) {
                            if (((v >> (8u * i)) & 0xFFu) == 0x7Fu) {
                                if (!flags_free) {
                                    flags_free = mbar_wait(acc_empty(set), (use - 1u) & 1u, abort_flag);
                                    if (!flags_free) {
                                        atomicOr(a.status, ST_WAIT_ACC);
                                        *abort_flag = 1;
                                    }
                                }
                                nan_rows[set * MQ_ROWS + row] = 1;
                                v &= ~(0xFFu << (8u * i));
                            }
                        }
                    }
                    *reinterpret_cast<uint32_t*>(smem + (sfa_of(s) - base) + 512u * q + (row & 31u) * 16u + (row >> 5) * 4u) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(prep_full(s));
            }
        }
        __syncwarp();
    } else if (warp < MQC_WARP_PIECE) {
        // ---------------------------------------------------------------- epilogue warps 10-13
        const uint32_t row = 32u * (warp & 3u) + lane;
        const uint32_t lane_base = tmem_base + ((32u * (warp & 3u)) << 16);
        bool alive = true;
        uint32_t j = 0;
        for (uint32_t ti = 0; ti < T && alive; ti++) {
            const uint32_t set = ti & 1u, use = ti >> 1;
            const uint32_t n0 = locate(ti, j);
            uint32_t go = 0;
            if (alive && lane == 0) go = mbar_wait(acc_full(set), use & 1u, abort_flag);
            go = __shfl_sync(0xFFFFFFFFu, go, 0);
            if (alive && !go) {
                if (lane == 0) {
                    atomicOr(a.status, ST_WAIT_ACC);
                    *abort_flag = 1;
                }
                alive = false;
            }
            if (!alive) break;
            tc_fence_after_sync();
            const MqChainJob& job = a.jobs[j];
            const bool in_n = n0 + row < job.n;
            const float g = in_n ? __ldg(job.wg + n0 + row) : 0.0f;
            const bool row_nan = nan_rows[set * MQ_ROWS + row] != 0;
            for (uint32_t t = 0; t < a.m; t++) {
                uint32_t d0[8], d1[8];
                tmem_ld_32x32b_x8(lane_base + set * TMEM_SET + 8u * t, d0);
                if (KB > 1u) tmem_ld_32x32b_x8(lane_base + set * TMEM_SET + ACC + 8u * t, d1);
                tmem_ld_wait();
                float v = 0.0f;
#pragma unroll
                for (int pc = 7; pc >= 0; pc--) {
                    float c = __uint_as_float(d0[pc]);
                    if (KB > 1u) c += __uint_as_float(d1[pc]);
                    v += c;
                }
                const uint32_t te = (PRE ? __ldg(job.pre_amax + t) : tok_amax[set * 4u + t]) >> 23;
                const float tscale = te >= 16u ? __uint_as_float((te - 8u) << 23) : 0.0f;
                v = v * tscale * g;
                if (row_nan || te == 255u) v = __uint_as_float(0x7FC00000u);
                const size_t o = (size_t)t * job.n + n0 + row;
                if (in_n) {
                    if (job.r) v += __ldcg(job.r + o);   // may be an earlier step's output
                    job.y[o] = v;
                }
            }
            nan_rows[set * MQ_ROWS + row] = 0;
            // the accumulators (and this set's flags) are free for the block's tile after next
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(set));

        }
    } else if (!PRE) {
        // ---------------------------------------------------------------- piece warps 14-17
        const uint32_t xw = warp - MQC_WARP_PIECE;
        const uint32_t xt = tid - 32u * MQC_WARP_PIECE;
        const uint32_t items = KB * a.m;
        const uint32_t PW = (S * a.m < MQC_PIECE_WARPS) ? S * a.m : MQC_PIECE_WARPS;
        for (uint32_t i = xt; i < S * (MQ_SF_BYTES / 16u); i += 32u * MQC_PIECE_WARPS) {
            const uint32_t s = i / (MQ_SF_BYTES / 16u), o = i % (MQ_SF_BYTES / 16u);
            *reinterpret_cast<uint4*>(smem + (sfb_of(s) - base) + 16u * o) = make_uint4(0, 0, 0, 0);
        }
        bool ok = true;          // a warp that gave up keeps walking the steps: barrier 4 below needs all four warps
        uint32_t j = 0;
        const void* prev_x = nullptr;
        for (uint32_t ti = 0; ti < T; ti++) {
            const uint32_t set = ti & 1u;
            locate(ti, j);
            const MqChainJob& job = a.jobs[j];
            // this block's epilogue of the tile before last is done with this set's slots (token maxima)
            if (ok && (ti >> 1) > 0u && !__all_sync(0xFFFFFFFFu, mbar_wait(acc_empty(set), ((ti >> 1) - 1u) & 1u, abort_flag))) {
                if (lane == 0) {
                    atomicOr(a.status, ST_WAIT_ACC);
                    *abort_flag = 1;
                }
                ok = false;
            }
            // the tokens' largest magnitudes (this set's slots were last read by this block's epilogue of the
            // tile before last, waited for above)
            asm volatile("bar.sync 4, %0;" ::"r"(32u * MQC_PIECE_WARPS) : "memory");
            if (*abort_flag) ok = false;
            // the same activations as the tile before (nothing in the run writes them): the other set's maxima hold
            const bool same_x = ti > 0u && job.x == prev_x;
            prev_x = job.x;
            if (xt < 4u) tok_amax[set * 4u + xt] = same_x ? tok_amax[(set ^ 1u) * 4u + xt] : 0u;
            asm volatile("bar.sync 4, %0;" ::"r"(32u * MQC_PIECE_WARPS) : "memory");
            if (ok && !same_x) {
                uint32_t mx[4] = {0, 0, 0, 0};
                const uint4* xr = reinterpret_cast<const uint4*>(job.x);
                const uint32_t row_chunks = XF32 ? a.k / 4u : a.k / 8u;
#pragma unroll 4
                for (uint32_t i = xt; i < row_chunks; i += 32u * MQC_PIECE_WARPS) {
                    uint4 v[4];
#pragma unroll
                    for (uint32_t t = 0; t < 4; t++)
                        v[t] = t < a.m ? __ldcg(xr + (size_t)t * row_chunks + i) : make_uint4(0, 0, 0, 0);
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
                    if (t < a.m) {
                        uint32_t r = mx[t];
                        if (!XF32) {
                            r = max(r & 0xFFFFu, r >> 16);
                            r = __float_as_uint(__half2float(__ushort_as_half((unsigned short)r)));
                        }
                        r = __reduce_max_sync(0xFFFFFFFFu, r);
                        if (lane == 0) atomicMax(tok_amax + set * 4u + t, r);
                    }
                }
            }
            asm volatile("bar.sync 4, %0;" ::"r"(32u * MQC_PIECE_WARPS) : "memory");
            for (uint32_t it = ((ok && xw < PW) ? xw : items); it < items; it += PW) {
                const uint32_t kb = it / a.m, tok = it - kb * a.m;
                const uint32_t gs = ti * KB + kb, s = gs % S, ph = (gs / S) & 1u;
                uint4 lo, hi = make_uint4(0, 0, 0, 0);
                if (XF32) {
                    const uint4* p4 = reinterpret_cast<const uint4*>(static_cast<const float*>(job.x) + (size_t)tok * a.k) +
                                      (size_t)kb * (MQ_STAGE_K / 4u) + 2u * lane;
                    lo = __ldcg(p4);
                    hi = __ldcg(p4 + 1);
                } else {
                    lo = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __half*>(job.x) + (size_t)tok * a.k) +
                                (size_t)kb * (MQ_STAGE_K / 8u) + lane);
                }
                const uint32_t te8 = tok_amax[set * 4u + tok] >> 23;
                uint32_t fb[8], w[8], e8;
                mq_widen<XF32>(lo, hi, fb);
                mq_digits(fb, w, e8);
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty(s), ph ^ 1u, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                uint8_t* const bt = smem + (b_of(s) - base) + (tok * MQ_PIECES) * 128u + 4u * (lane & 3u);
#pragma unroll
                for (uint32_t pc = 0; pc < MQ_PIECES; pc++)
                    *reinterpret_cast<uint32_t*>(bt + pc * 128u + (((lane >> 2) ^ pc) << 4)) = w[pc];
                const int q0 = 8 - (int)(te8 - e8);
                const uint32_t grp = lane >> 1;
                uint8_t* const sb = smem + (sfb_of(s) - base);
#pragma unroll
                for (uint32_t i = 0; i < 4; i++) {
                    const uint32_t pc = 4u * (lane & 1u) + i;
                    sb[mq_sfb_offset(tok * MQ_PIECES + pc, grp, false)] = (uint8_t)mq_ue4m3_pow2(q0 - 2 * (int)pc);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(prep_full(s));
            }
        }
        __syncwarp();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, MQ_TMEM_COLS);
    }
}

}  // namespace lexb
