// gemm_fp4 for m > 256 on sm_100a: the two-CTA form of gemm_fp4_sm100.cuh.
//
// The cost of a tile is the FP4 decode, not the multiply (the reference found the same on Ada,
// crates/lex-msl/src/gemm.rs:107-110), so every weight should be decoded once for as many
// tokens as possible.  A pair of CTAs (one cluster, two SMs) owns 256 rows of W and 512
// tokens: each CTA decodes its own 128 rows once per K step, each loads half of the x tile
// (two blocks of 128 tokens), and the leader CTA issues tcgen05.mma.cta_group::2 - M = 256
// rows of W (128 from each CTA's shared memory), N = 256 tokens (128 from each) - twice per
// 16 columns of K, once per token block.  Each CTA's TMEM then holds its 128 weight rows x 512
// tokens (all 512 columns).  Per CTA and K step of 64 that is 1024 tensor-core clocks for 8192
// decoded weights: twice the decode budget of the one-CTA kernel, and half its shared-memory
// traffic for x.
//
// Barriers: the leader CTA's `x_full` and `w_full` collect arrivals from both CTAs (the partner
// arrives through shared::cluster addresses; its TMA reports bytes to the leader's barrier);
// `empty` and `acc_full` exist in both CTAs and are signalled together by tcgen05.commit.
// No TMA multicast is used.
#pragma once
#include "fp4_decode.cuh"
#include "gemm_fp4_sm100.cuh"
#include "sm100_ptx.cuh"

namespace lexb {

constexpr uint32_t PAIR_TOKENS = 512;                 // tokens per pair tile
constexpr uint32_t PAIR_XBLK_ROWS = 128;              // tokens per TMA box (one CTA's half of a block)
constexpr uint32_t PAIR_XBLK_BYTES = PAIR_XBLK_ROWS * 128u;                  // 16 KiB
constexpr uint32_t PAIR_STAGE_BYTES = 2u * PAIR_XBLK_BYTES + GEMM_W_TILE_BYTES;   // 48 KiB
constexpr uint32_t PAIR_TMEM_COLS = 512;

__host__ __device__ constexpr uint32_t pair_smem_bytes(uint32_t stages) {
    return stages * PAIR_STAGE_BYTES + (3u * stages + 1u) * 8u + 16u + 1024u;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_fp4_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);

    const uint32_t S = a.stages;
    const uint32_t bars = base + S * PAIR_STAGE_BYTES;
    auto x_full = [&](uint32_t s) { return bars + 8u * s; };            // used in the leader only
    auto w_full = [&](uint32_t s) { return bars + 8u * (S + s); };      // used in the leader only
    auto empty = [&](uint32_t s) { return bars + 8u * (2u * S + s); };  // both CTAs
    const uint32_t acc_full = bars + 8u * 3u * S;                       // both CTAs
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(smem + S * PAIR_STAGE_BYTES + (3u * S + 1u) * 8u);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t m_tile = pair % a.m_tiles, n_pair = pair / a.m_tiles;
    const uint32_t m0 = m_tile * PAIR_TOKENS;
    const uint32_t n0 = n_pair * 2u * GEMM_TN + rank * GEMM_TN;
    const uint32_t KB = a.k / GEMM_BK;

    if (tid == 0) {
        *abort_flag = 0;
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(x_full(s), 2);                         // one arrive.expect_tx per CTA
            mbar_init(w_full(s), 16);                        // one arrive per dequant warp of either CTA
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
    }
    if (warp == GEMM_WARP_TMA && lane == 0) prefetch_tensormap(&tmap_x);
    if (warp == GEMM_WARP_MMA) {
        tmem_alloc_pair(smem_u32(tmem_slot), PAIR_TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                                      // both CTAs' barriers exist before any remote arrive
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == GEMM_WARP_TMA) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            for (uint32_t kb = 0; kb < KB; kb++) {
                const uint32_t s = kb % S, ph = (kb / S) & 1u;
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t lead_bar = map_to_cta(x_full(s), 0);
                mbar_arrive_expect_tx_cluster(lead_bar, 2u * PAIR_XBLK_BYTES);
                const uint32_t dst = base + s * PAIR_STAGE_BYTES;
                // token block tb covers tokens m0 + 256 tb .. +255; this CTA holds 128 of them
                tma_load_2d_pair(dst, &tmap_x, (int)(kb * GEMM_BK), (int)(m0 + rank * PAIR_XBLK_ROWS), lead_bar);
                tma_load_2d_pair(dst + PAIR_XBLK_BYTES, &tmap_x, (int)(kb * GEMM_BK),
                                 (int)(m0 + 256u + rank * PAIR_XBLK_ROWS), lead_bar);
            }
            if (*abort_flag) {
                // The byte counts of this CTA's copies are kept by the leader's barriers, which
                // the partner cannot poll: give copies still in flight a fixed, bounded time to land.
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) {
                }
            }
        }
        __syncwarp();
    } else if (warp == GEMM_WARP_MMA) {
        // ---------------------------------------------------------------- MMA issuer (leader only)
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = umma_idesc_f16_f32(256u, 256u);
            bool ok = true;
            for (uint32_t kb = 0; kb < KB; kb++) {
                const uint32_t s = kb % S, ph = (kb / S) & 1u;
                if (!mbar_wait_cluster(x_full(s), ph, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_X_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                if (!mbar_wait_cluster(w_full(s), ph, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_W_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t x_addr = base + s * PAIR_STAGE_BYTES;
                const uint32_t w_addr = x_addr + 2u * PAIR_XBLK_BYTES;
#pragma unroll
                for (uint32_t kk = 0; kk < GEMM_BK / 16; kk++) {
                    const uint64_t a_desc = umma_desc_k_sw128(w_addr + kk * 32u);
                    const uint32_t acc = (kb | kk) != 0u;
                    umma_f16_ss_pair(tmem_base, a_desc, umma_desc_k_sw128(x_addr + kk * 32u), idesc, acc);
                    umma_f16_ss_pair(tmem_base + 256u, a_desc, umma_desc_k_sw128(x_addr + PAIR_XBLK_BYTES + kk * 32u),
                                     idesc, acc);
                }
                umma_commit_pair(empty(s), 3);               // frees the stage in both CTAs
            }
            if (ok) umma_commit_pair(acc_full, 3);
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- dequant warps 0-7 (both CTAs)
        // Thread (row r, half h): a warp covers 32 consecutive rows and one half, so the eight
        // 16-byte chunks any 8 consecutive lanes store fall into eight different bank groups.
        const uint32_t r = tid & 127u, h = tid >> 7;
        const uint32_t row = n0 + r;
        const float g = __ldg(a.wg + row);
        const uint4* qrow = reinterpret_cast<const uint4*>(a.wq + (size_t)row * (a.k / 2)) + h;
        const uint32_t* srow = reinterpret_cast<const uint32_t*>(a.ws + (size_t)row * (a.k / 16));
        const uint32_t w_off = 2u * PAIR_XBLK_BYTES + r * 128u;
        const uint32_t sw_xor = r & 7u;
        const uint32_t c = 4u * h;
        // two K steps of codes and scales in flight
        uint4 q0 = __ldg(qrow), q1 = KB > 1 ? __ldg(qrow + 2) : make_uint4(0, 0, 0, 0);
        uint32_t s0 = __ldg(srow), s1 = KB > 1 ? __ldg(srow + 1) : 0u;
        bool ok = true;
        for (uint32_t kb = 0; kb < KB; kb++) {
            const uint32_t s = kb % S, ph = (kb / S) & 1u;
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
            if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
                atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                *abort_flag = 1;
                ok = false;
                break;
            }
            uint8_t* wt = smem + s * PAIR_STAGE_BYTES + w_off;
            *reinterpret_cast<uint4*>(wt + (((c + 0u) ^ sw_xor) << 4)) = o0;
            *reinterpret_cast<uint4*>(wt + (((c + 1u) ^ sw_xor) << 4)) = o1;
            *reinterpret_cast<uint4*>(wt + (((c + 2u) ^ sw_xor) << 4)) = o2;
            *reinterpret_cast<uint4*>(wt + (((c + 3u) ^ sw_xor) << 4)) = o3;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(w_full(s), 0));
        }
        __syncwarp();
        // ---------------------------------------------------------------- epilogue (both CTAs)
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
            for (uint32_t cc = half; cc < PAIR_TOKENS / 16u; cc += 2u) {
                const uint32_t t0 = m0 + cc * 16u;
                if (t0 >= a.m) break;                        // warp-uniform
                uint32_t v[16];
                tmem_ld_32x32b_x16(tmem_base + ((32u * quarter) << 16) + cc * 16u, v);
                tmem_ld_wait();
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
    cluster_sync_all();          // the partner's shared memory and barriers stay alive until both are done
    if (warp == GEMM_WARP_MMA) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
    }
}

}  // namespace lexb
