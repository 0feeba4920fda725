// gemm_fp4 for m > 8 on sm_100a: the two-CTA form of gemm_fp4_sm100.cuh.
//
// The cost of a tile is the FP4 decode, not the multiply (the reference found the same on Ada,
// crates/lex-msl/src/gemm.rs:107-110), so every weight should be decoded once for as many
// tokens as possible.  A pair of CTAs (one cluster, two SMs) owns 256 rows of W and up to 512
// tokens: each CTA decodes its own 128 rows once per K step, each loads half of the x tile
// (two blocks of 128 tokens), and the leader CTA issues tcgen05.mma.cta_group::2 - M = 256
// rows of W (128 from each CTA), N = 256 tokens (128 from each) - twice per 16 columns of K,
// once per token block.  Each CTA's TMEM then holds its 128 weight rows x 512 tokens (all 512
// columns).  Per CTA and K step of 64 that is 1024 tensor-core clocks for 8192 decoded weights:
// twice the decode budget of the one-CTA kernel, and half its shared-memory traffic for x.
//
// Smaller tiles have one token block of 256, 128 or 64 tokens (N of the MMAs; each CTA holds
// half).  Their decoded W tiles go to tensor memory instead of shared memory - the accumulator
// leaves at least 256 of the 512 columns free - and the MMAs take their A operand from there;
// a ring stage then holds two K steps.
//
// The packed weights never pass through a dequant thread's global loads: a third single-thread
// role brings them in by TMA, 256 columns of K at a time (a [128 rows x 128 bytes] tile of codes,
// 128-byte swizzled, and a [128 x 16 bytes] tile of scales), two or three such blocks in flight,
// and a dequant thread reads its row's 32 bytes of codes and 4 scale bytes of a K step from
// shared memory.
//
// Barriers: the MMA warp's own loop sets the pace of a K step when the MMAs are short (every wait it
// makes costs about a hundred cycles even when the barrier is ready, every commit more), so a ring
// stage has ONE barrier the MMA warp waits on and ONE it signals.  `full[j]` (leader CTA) collects
// everything stage step j needs: the two x producers' arrive.expect_tx (the partner's through a
// shared::cluster address; its TMA reports bytes to the leader's barrier), the four warps of each
// decode group of the leader that owns a K step of it, and one arrival from the partner's relay
// thread, which waits on the partner's own `w_part` barrier for its warps.  `done[j]` exists in both
// CTAs and is signalled in both by one tcgen05.commit: it frees the x stage and the W stage of step j
// at once.  Both rings of barriers are indexed by step modulo max(x stages, W stages, 4); the data
// rings keep their own depths.  No TMA multicast is used.
#pragma once
#include "fp4_decode.cuh"
#include "gemm_fp4_sm100.cuh"
#include "sm100_ptx.cuh"

namespace lexb {

constexpr uint32_t PAIR_TOKENS = 512;                 // tokens of the largest pair tile
constexpr uint32_t PAIR_XBLK_ROWS = 128;              // tokens per TMA box (one CTA's half of a block)
constexpr uint32_t PAIR_XBLK_BYTES = PAIR_XBLK_ROWS * 128u;                  // 16 KiB
// a stage of the x ring holds this CTA's half of one token block (tiles of 256 tokens) or of two (512): 16 or 32 KiB
// (`k_sub` K steps of 64 columns per stage: 1, or 2 with the W tiles in tensor memory)
// (`x_rows`: tokens each CTA holds of a token block - 128, or 64 / 32 with tiles of 128 / 64 tokens)
__host__ __device__ constexpr uint32_t pair_x_stage_bytes(uint32_t tok_blocks, uint32_t k_sub = 1, uint32_t x_rows = PAIR_XBLK_ROWS) {
    return tok_blocks * k_sub * x_rows * 128u;
}
// The epilogue stages its chunks in the first 64 KiB of the rings (idle by then); the barriers sit behind.
constexpr uint32_t PAIR_STAGING_BYTES = 65536;
constexpr uint32_t PAIR_TMEM_COLS = 512;
constexpr uint32_t PAIR_DEQ_THREADS = 512;            // 16 warps in 4 groups: a group decodes one K step in four, a row per thread
constexpr uint32_t PAIR_WARP_TMA = 16;
constexpr uint32_t PAIR_WARP_MMA = 17;                // leader: issues the MMAs; partner: relays its w_full
constexpr uint32_t PAIR_WARP_RAW = 18;                // TMA of the packed codes and scales
constexpr uint32_t PAIR_THREADS = 608;
constexpr uint32_t PAIR_RAW_K = 256;                  // K columns per block of packed weights
constexpr uint32_t PAIR_RAW_WQ_BYTES = GEMM_TN * (PAIR_RAW_K / 2);          // 16 KiB
constexpr uint32_t PAIR_RAW_WS_BYTES = GEMM_TN * (PAIR_RAW_K / 16);         // 2 KiB
constexpr uint32_t PAIR_RAW_BYTES = PAIR_RAW_WQ_BYTES + PAIR_RAW_WS_BYTES;
constexpr uint32_t PAIR_RAW_STAGES = 2;                // default depth of the ring of packed-weight blocks

// x ring, W ring (their depths are independent: the decoded W tiles may run further ahead of the
// MMA than the x tiles), packed-weight blocks, barriers, TMEM slot + abort flag, alignment slack
// (`w_in_tmem`: the decoded W tiles live in tensor memory and take no shared memory)
__host__ __device__ constexpr uint32_t pair_smem_bytes(uint32_t tok_blocks, uint32_t sx, uint32_t sw, uint32_t sr = PAIR_RAW_STAGES,
                                                      bool w_in_tmem = false, uint32_t k_sub = 1, uint32_t x_rows = PAIR_XBLK_ROWS) {
    const uint32_t rings = sx * pair_x_stage_bytes(tok_blocks, k_sub, x_rows) + (w_in_tmem ? 0u : sw * GEMM_W_TILE_BYTES) + sr * PAIR_RAW_BYTES;
    return (rings > PAIR_STAGING_BYTES ? rings : PAIR_STAGING_BYTES) +
           (2u * sx + 3u * sw + 1u + 2u * sr) * 8u + 16u + 1024u;
}

template <bool TRACE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_fp4_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_wq,
                             const __grid_constant__ CUtensorMap tmap_ws, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw_addr);

    const uint32_t SX = a.stages, SW = a.w_stages, SR = a.raw_stages;
    const uint32_t KS = a.k_sub;                                           // K steps per ring stage: 1, or 2 (W in TMEM only)
    const uint32_t XR = a.x_rows;                                          // tokens this CTA holds of a token block
    const uint32_t XB = XR * 128u;                                         // bytes of one x box: XR tokens x 64 K columns
    const uint32_t XSB = pair_x_stage_bytes(a.tok_blocks, KS, XR);
    const uint32_t w_base = base + SX * XSB;                               // decoded W tiles
    // Flag bit 2 (tiles of 256 tokens only): the decoded W tiles go to tensor memory - columns 256.. of this CTA's
    // TMEM, 32 columns per K step (so at most 8 K steps in flight), the accumulator keeps columns 0-255 - and the
    // MMAs take their A operand from there.  With 256 tokens a K step is bound by the shared-memory pipe; this takes the W
    // tile's 16 KiB of stores and 16 KiB of operand reads per K step off it, and the W ring out of shared memory.
    // One accumulator instead of two.  What then sets the pace is the MMA warp's own loop (a wait, a fence, a commit:
    // ~600 cycles next to four decode warps on its scheduler, against 512 for the four MMAs of a K step), so in this
    // mode a ring stage may hold two K steps (k_sub = 2): two decode groups fill one stage and that loop runs half as
    // often.
    const bool w_tmem = (a.flags & 4u) != 0u && a.tok_blocks == 1u;
    const uint32_t a_col0 = XR <= 64u ? 128u : 256u;                       // first TMEM column of the W ring: behind the accumulator
    const uint32_t raw_base = w_base + (w_tmem ? 0u : SW * GEMM_W_TILE_BYTES);     // packed weight blocks
    const uint32_t rings_end = raw_base + SR * PAIR_RAW_BYTES;
    const uint32_t bars = rings_end > base + PAIR_STAGING_BYTES ? rings_end : base + PAIR_STAGING_BYTES;
    // Depth of the barrier rings: no data ring may be deeper, and at least 4 - a decode group visits the `done`
    // ring every fourth K step (every 4 / KS stage steps), and a parity wait is only right if the barrier cannot be
    // two phases behind the one awaited: the group's previous wait (step j - 4 / KS) guarantees phase (j - DN) only
    // if DN >= 4 / KS.
    const uint32_t DN = (SX > SW ? SX : SW) > 4u ? (SX > SW ? SX : SW) : 4u;
    auto full = [&](uint32_t j) { return bars + 8u * j; };                        // leader only: all inputs of K step j
    auto done = [&](uint32_t j) { return bars + 8u * (DN + j); };                 // both CTAs: K step j's MMAs complete
    auto w_part = [&](uint32_t s) { return bars + 8u * (2u * DN + s); };          // partner only: its own decode warps
    const uint32_t nb = 2u * DN + SW;
    const uint32_t acc_full = bars + 8u * nb;                                     // both CTAs
    auto raw_full = [&](uint32_t rs) { return bars + 8u * (nb + 1u + rs); };
    auto raw_empty = [&](uint32_t rs) { return bars + 8u * (nb + 1u + SR + rs); };
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(smem + (bars - base) + (nb + 1u + 2u * SR) * 8u);
    volatile uint32_t* const abort_flag = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t split = pair % a.k_splits, tile = pair / a.k_splits;
    const uint32_t m_tile = tile % a.m_tiles, n_pair = tile / a.m_tiles;
    const uint32_t TB = a.tok_blocks;                              // 1 or 2 blocks of 256 tokens per tile
    const uint32_t m0 = m_tile * TB * 2u * XR;                     // TB = 2 only with XR = 128
    const uint32_t n0 = n_pair * 2u * GEMM_TN + rank * GEMM_TN;     // may be == n in the last pair: nothing to store
    const uint32_t kb0 = split * a.kb_per_split;                    // first K step of this split (a multiple of 4)
    const uint32_t kb_all = a.k / GEMM_BK;
    const uint32_t KB = (kb_all - kb0 < a.kb_per_split) ? (kb_all - kb0) : a.kb_per_split;
    const long long t_start = clock64();
    unsigned long long gt_start = 0;
    if (TRACE) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt_start));

    if (tid == 0) {
        *abort_flag = 0;
        for (uint32_t j = 0; j < DN; j++) {
            // one arrive.expect_tx per CTA, one arrival per warp of the leader's decode group, one from the partner's relay
            mbar_init(full(j), 2u + KS * (PAIR_DEQ_THREADS / 128u) + 1u);
            mbar_init(done(j), 1);
        }
        for (uint32_t s = 0; s < SW; s++) mbar_init(w_part(s), KS * (PAIR_DEQ_THREADS / 128u));
        for (uint32_t rs = 0; rs < SR; rs++) {
            mbar_init(raw_full(rs), 1);
            mbar_init(raw_empty(rs), PAIR_DEQ_THREADS / 32u);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
    }
    if (warp == PAIR_WARP_TMA && lane == 0) prefetch_tensormap(&tmap_x);
    if (warp == PAIR_WARP_RAW && lane == 0) {
        prefetch_tensormap(&tmap_wq);
        prefetch_tensormap(&tmap_ws);
    }
    if (warp == PAIR_WARP_MMA) {
        tmem_alloc_pair(smem_u32(tmem_slot), PAIR_TMEM_COLS);
        tmem_relinquish_pair();
    }
    allow_dependents();                                      // the next launch may be scheduled as SMs free up
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                                      // both CTAs' barriers exist before any remote arrive
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this block's shared memory and TMEM.  From here on the kernel
    // reads x, the weights and r and writes y: wait for the launch ahead of this one in the stream.
    // With flag bit 1 (the packed weights are known to be constant: declared by the caller or proven from
    // the step list) the two roles that touch only wq, ws and wg - the copy of the packed weights and the
    // decode into shared memory - start at once and fill their rings while the launch ahead still runs;
    // each joins the stream's order before its first wait on a ring slot (a bounded wait must not run
    // against another launch's time) and, for the decode warps, before the epilogue.
    const bool early_w = (a.flags & 2u) != 0u;

    const bool weight_role = warp == PAIR_WARP_RAW || warp < PAIR_DEQ_THREADS / 32u;
    if (!(early_w && weight_role)) grid_dependency_wait();

    if (warp == PAIR_WARP_TMA) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            RingPos px, pf, pe;              // x stage, barrier of this K step, barrier of the K step that held the stage
            for (uint32_t st = 0; st < KB / KS; st++, px.advance(SX), pf.advance(DN)) {
                const uint32_t s = px.s;
                if (st >= SX) {
                    if (!mbar_wait(done(pe.s), pe.ph, abort_flag)) {
                        atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                        *abort_flag = 1;
                        break;
                    }
                    pe.advance(DN);
                }
                const uint32_t lead_bar = map_to_cta(full(pf.s), 0);
                mbar_arrive_expect_tx_cluster(lead_bar, KS * TB * a.x_tx_bytes);
                const uint32_t dst = base + s * XSB;
                const uint32_t kb = kb0 + st * KS;
                // token block tb covers tokens m0 + 256 tb .. +255; this CTA holds 128 of them
                tma_load_2d_pair(dst, &tmap_x, (int)(kb * GEMM_BK), (int)(m0 + rank * XR), lead_bar);
                if (TB > 1u)
                    tma_load_2d_pair(dst + XB, &tmap_x, (int)(kb * GEMM_BK), (int)(m0 + 2u * XR + rank * XR), lead_bar);
                for (uint32_t sub = 1; sub < KS; sub++)      // the stage's further K steps (one token block)
                    tma_load_2d_pair(dst + sub * XB, &tmap_x, (int)((kb + sub) * GEMM_BK), (int)(m0 + rank * XR), lead_bar);
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
    } else if (warp == PAIR_WARP_RAW) {
        // ---------------------------------------------------------------- TMA of packed weights (both CTAs)
        if (lane == 0) {
            const uint32_t RB = (KB + 3u) / 4u, rb0 = kb0 / 4u;
            RingPos pr;
            for (uint32_t rb = 0; rb < RB; rb++, pr.advance(SR)) {
                const uint32_t rs = pr.s, ph = pr.ph;
                if (early_w && rb == SR) grid_dependency_wait();     // the ring is full: join the stream's order
                if (!mbar_wait(raw_empty(rs), ph ^ 1u, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_EMPTY_TMA);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_expect_tx(raw_full(rs), PAIR_RAW_BYTES);
                const uint32_t dst = raw_base + rs * PAIR_RAW_BYTES;
                tma_load_2d(dst, &tmap_wq, (int)((rb0 + rb) * (PAIR_RAW_K / 2)), (int)n0, raw_full(rs));
                tma_load_2d(dst + PAIR_RAW_WQ_BYTES, &tmap_ws, (int)((rb0 + rb) * (PAIR_RAW_K / 16)), (int)n0, raw_full(rs));
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) {
                }
            }
        }
        __syncwarp();
    } else if (warp == PAIR_WARP_MMA) {
        if (rank != 0 && lane == 0) {
            // ------------------------------------------------------------ partner: relay of its W tiles
            // One cluster-scope arrive per K step from this otherwise idle thread, so that the
            // dequant threads only ever touch barriers of their own CTA.
            RingPos pw, pf;
            for (uint32_t st = 0; st < KB / KS; st++, pw.advance(SW), pf.advance(DN)) {
                if (!mbar_wait(w_part(pw.s), pw.ph, abort_flag)) {
                    atomicOr(a.status, ST_WAIT_W_FULL);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_cluster(map_to_cta(full(pf.s), 0));
            }
        }
        // ---------------------------------------------------------------- MMA issuer (leader only)
        // The whole warp runs the loop with warp-uniform values; one elected lane issues.
        if (rank == 0) {
            const uint32_t idesc = umma_idesc_f16_f32(256u, 2u * XR);       // N = the tokens of one block, both CTAs' halves
            const uint32_t x_lo0 = umma_desc_lo(base), w_lo0 = umma_desc_lo(w_base);
            const uint32_t d0 = tmem_base, d1 = tmem_base + 256u;
            const bool reuse_a = (a.flags & 1u) != 0u;
            bool ok = true;
            long long wait_full = 0, t_first = 0, t_issue = 0;
            RingPos px, pw, pf;
            for (uint32_t kb = 0; kb < KB; kb += KS, px.advance(SX), pw.advance(SW), pf.advance(DN)) {
                const uint32_t s = px.s, sw = pw.s;
                long long tw0 = 0;
                if (TRACE) tw0 = clock64();
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(full(pf.s), pf.ph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_X_FULL | ST_WAIT_W_FULL);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                if (TRACE) {
                    const long long tw3 = clock64();
                    wait_full += tw3 - tw0;
                    if (kb == 0) t_first = tw3;
                }
                tc_fence_after_sync();
                long long ti0 = 0;
                if (TRACE) ti0 = clock64();
                // low descriptor halves of this K step's tiles; +2 per 16 columns of K
                const uint32_t b0 = x_lo0 + s * (XSB >> 4);
                const uint32_t b1 = b0 + (XB >> 4);
                const uint32_t aw = w_lo0 + sw * (GEMM_W_TILE_BYTES >> 4);
                if (elect_one()) {
                if (TB > 1u) {
                    const uint32_t first = kb != 0u;      // the very first MMA of each block overwrites
                    if (reuse_a) {
                        // both token blocks multiply the same W tile: read it from shared memory once
                        umma2_flag_fill(d0, aw, b0, idesc, first);
                        umma2_flag_lastuse(d1, aw, b1, idesc, first);
#pragma unroll
                        for (uint32_t kk = 1; kk < GEMM_BK / 16; kk++) {
                            umma2_acc_fill(d0, aw + 2u * kk, b0 + 2u * kk, idesc);
                            umma2_acc_lastuse(d1, aw + 2u * kk, b1 + 2u * kk, idesc);
                        }
                    } else {
                        umma2_flag(d0, aw, b0, idesc, first);
                        umma2_flag(d1, aw, b1, idesc, first);
#pragma unroll
                        for (uint32_t kk = 1; kk < GEMM_BK / 16; kk++) {
                            umma2_acc(d0, aw + 2u * kk, b0 + 2u * kk, idesc);
                            umma2_acc(d1, aw + 2u * kk, b1 + 2u * kk, idesc);
                        }
                    }
                } else if (w_tmem) {
                    const uint32_t at = tmem_base + a_col0 + sw * (32u * KS);
                    umma2_ts_flag(d0, at, b0, idesc, kb != 0u);
#pragma unroll
                    for (uint32_t kk = 1; kk < GEMM_BK / 16; kk++) umma2_ts_flag(d0, at + 8u * kk, b0 + 2u * kk, idesc, 1u);
                    for (uint32_t sub = 1; sub < KS; sub++) {      // the stage's further K steps: the next 32 columns, the next x block
                        const uint32_t as = at + 32u * sub, bs = b0 + sub * (XB >> 4);
#pragma unroll
                        for (uint32_t kk = 0; kk < GEMM_BK / 16; kk++) umma2_ts_flag(d0, as + 8u * kk, bs + 2u * kk, idesc, 1u);
                    }
                } else {
                    // one token block: even and odd K steps go to two accumulators, which halves the
                    // run of truncating f32 additions each one sees
                    const uint32_t d = (kb & 1u) ? d1 : d0;
                    umma2_flag(d, aw, b0, idesc, kb >= 2u);
#pragma unroll
                    for (uint32_t kk = 1; kk < GEMM_BK / 16; kk++) umma2_acc(d, aw + 2u * kk, b0 + 2u * kk, idesc);
                }
                umma_commit_pair(done(pf.s), 3);             // frees this K step's x stage and W stage in both CTAs
                }
                __syncwarp();
                if (TRACE) t_issue += clock64() - ti0;
            }
            if (ok && elect_one()) umma_commit_pair(acc_full, 3);
            __syncwarp();
            if (TRACE && a.trace && lane == 0) {
                unsigned long long* tr = a.trace + 16ull * blockIdx.x;
                tr[1] = (unsigned long long)t_first;      // first stage ready
                tr[2] = (unsigned long long)clock64();    // all MMAs issued
                tr[3] = (unsigned long long)wait_full;    // cycles the MMA warp waited for a K step's inputs
                tr[4] = 0;
                tr[5] = 0;
                tr[11] = (unsigned long long)t_issue;     // cycles spent issuing MMAs (queue back-pressure included)
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- dequant warps 0-15 (both CTAs)
        // Four groups of four warps.  A group decodes WHOLE K steps: of every block of 256 K columns, group q takes
        // K step q - its 128 threads one row each, 64 weights per thread - so a warp meets the barriers once per four
        // K steps (one wait for the packed block, one for a free W stage, one proxy fence, one arrival) where a
        // split of every K step over all 16 warps met them every K step; those waits, not the decode arithmetic,
        // were the longer part of a warp's loop.  The four groups work on four consecutive K steps at once, and
        // each scheduler holds one warp of every group.
        // Thread (row r, K step q of the block): a warp covers 32 consecutive rows, so the 16-byte chunks any 8
        // consecutive lanes load or store fall into different bank groups.
        const uint32_t r = tid & 127u, q = tid >> 7;
        const uint32_t row = n0 + r;
        // rows past n (second half of an odd last pair): the copy engine fills their codes with zeros
        const float g = row < a.n ? __ldg(a.wg + row) : 0.0f;
        const uint32_t w_off = (w_base - base) + r * 128u;
        const uint32_t sw_xor = r & 7u;
        const uint8_t* raw0 = smem + (raw_base - base);
        bool ok = true;
        long long dq_wait_raw = 0, dq_wait_empty = 0, dq_t0 = 0;
        if (TRACE) dq_t0 = clock64();
        RingPos pr, pw, pf, pe;          // packed block; W stage and barrier of this K step; barrier of the stage's last user
        pw.seek(q / KS, SW);
        pf.seek(q / KS, DN);
        const uint32_t hop = 4u / KS;                                // stage steps between this group's K steps
        const uint32_t sub_col = (q % KS) * 32u;                     // this group's K step within a two-step stage
        bool joined = !early_w, pe_set = false;
        for (uint32_t kb = q; kb < KB; kb += 4u, pr.advance(SR), pw.advance_by(hop, SW), pf.advance_by(hop, DN)) {
            const uint32_t rs = pr.s, rph = pr.ph;
            long long tq0 = 0;
            if (TRACE) tq0 = clock64();
            // waits are made warp-uniform (a vote) so that a give-up leaves no lane behind at a __syncwarp
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(raw_full(rs), rph, abort_flag))) {
                atomicOr(a.status, ST_WAIT_X_FULL);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (TRACE) dq_wait_raw += clock64() - tq0;
            // this K step's 32 bytes of codes (chunks 2q, 2q + 1 of the row, in the swizzled tile) and 4 scale bytes
            const uint8_t* raw = raw0 + rs * PAIR_RAW_BYTES;
            const uint4 c0 = *reinterpret_cast<const uint4*>(raw + r * 128u + (((2u * q) ^ sw_xor) << 4));
            const uint4 c1 = *reinterpret_cast<const uint4*>(raw + r * 128u + (((2u * q + 1u) ^ sw_xor) << 4));
            const uint32_t sc = *reinterpret_cast<const uint32_t*>(raw + PAIR_RAW_WQ_BYTES + r * 16u + 4u * q);
            __syncwarp();
            if (lane == 0) mbar_arrive(raw_empty(rs));                   // this warp is done with the block
            uint4 o[8];
            decode_group16(make_uint2(c0.x, c0.y), sc & 0xFFu, g, o[0], o[1]);
            decode_group16(make_uint2(c0.z, c0.w), (sc >> 8) & 0xFFu, g, o[2], o[3]);
            decode_group16(make_uint2(c1.x, c1.y), (sc >> 16) & 0xFFu, g, o[4], o[5]);
            decode_group16(make_uint2(c1.z, c1.w), sc >> 24, g, o[6], o[7]);
            long long tq1 = 0;
            if (TRACE) tq1 = clock64();
            const uint32_t st = kb / KS;                                 // KS is 1 or 2
            if (st >= SW) {
                if (!joined) {                                           // first wait on a W stage: join the stream's order
                    grid_dependency_wait();
                    joined = true;
                }
                if (!pe_set) {
                    pe.seek(st - SW, DN);
                    pe_set = true;
                }
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(done(pe.s), pe.ph, abort_flag))) {
                    atomicOr(a.status, ST_WAIT_EMPTY_DEQ);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                pe.advance_by(hop, DN);
            }
            if (TRACE) dq_wait_empty += clock64() - tq1;
            if (w_tmem) {
                // this lane's row of the tile: 64 f16 in K order = 32 columns of its TMEM lane
                uint32_t v[32];
#pragma unroll
                for (uint32_t c = 0; c < 8; c++) {
                    v[4u * c + 0u] = o[c].x;
                    v[4u * c + 1u] = o[c].y;
                    v[4u * c + 2u] = o[c].z;
                    v[4u * c + 3u] = o[c].w;
                }
                tmem_st_32x32b_x32(tmem_base + ((32u * (warp & 3u)) << 16) + a_col0 + pw.s * (32u * KS) + sub_col, v);
                tmem_st_wait();
                tc_fence_before_sync();
            } else {
                uint8_t* const wt = smem + pw.s * GEMM_W_TILE_BYTES + w_off;
#pragma unroll
                for (uint32_t c = 0; c < 8; c++) *reinterpret_cast<uint4*>(wt + ((c ^ sw_xor) << 4)) = o[c];
                fence_proxy_async_smem();       // generic-proxy stores -> visible to the MMA's reads
            }
            // One arrival per warp: hundreds of arrivals on one barrier serialise in shared memory.  The tile is
            // reported to the K step's barrier (leader) or to the relay's (partner).
            __syncwarp();
            if (lane == 0) mbar_arrive(rank == 0u ? full(pf.s) : w_part(pw.s));
        }
        if (TRACE && a.trace && (tid == 0 || tid == 511)) {
            unsigned long long* tr = a.trace + 16ull * blockIdx.x + (tid == 0 ? 8 : 12);
            tr[0] = (unsigned long long)(clock64() - dq_t0);     // dequant loop, total
            tr[1] = (unsigned long long)dq_wait_raw;            // ... of which waiting for packed weights
            tr[2] = (unsigned long long)dq_wait_empty;          // ... and for a free W stage
        }
        __syncwarp();
        // ---------------------------------------------------------------- epilogue (both CTAs)
        if (early_w) grid_dependency_wait();        // r, y and the partials belong to the stream's order
        uint32_t go = 0;
        if (lane == 0) {
            go = ok && mbar_wait(acc_full, 0, abort_flag);
            if (!go) {
                atomicOr(a.status, ST_WAIT_ACC);
                *abort_flag = 1;
            }
        }
        go = __shfl_sync(0xFFFFFFFFu, go, 0);
        if (TRACE && a.trace && tid == 0) {
            a.trace[16ull * blockIdx.x + 0] = (unsigned long long)t_start;
            // block start on the global timer (ns): in the partner's record (the leader's slot 11 holds its MMA issue cycles)
            if (rank != 0u) a.trace[16ull * blockIdx.x + 11] = gt_start;
            a.trace[16ull * blockIdx.x + 6] = (unsigned long long)clock64();   // accumulator complete
        }
        if (go && n0 < a.n) {
            tc_fence_after_sync();
            const uint32_t quarter = warp & 3u, slice = warp >> 2;      // 4 lane quarters x 4 column slices
            const bool to_partial = a.k_splits > 1u;
            float* const out = to_partial ? a.partial + (size_t)split * a.m * a.n : a.y;
            const float* const res = to_partial ? nullptr : a.r;
            const bool two_acc = TB == 1u && KB > 1u && !w_tmem;
            for (uint32_t cc = slice; cc < TB * XR / 8u; cc += 4u) {     // chunks of 16 tokens: 2 XR tokens per block
                const uint32_t t0 = m0 + cc * 16u;
                if (t0 >= a.m) break;                        // warp-uniform
                uint32_t v[16];
                tmem_ld_32x32b_x16(tmem_base + ((32u * quarter) << 16) + cc * 16u, v);
                if (two_acc) {
                    uint32_t v2[16];
                    tmem_ld_32x32b_x16(tmem_base + ((32u * quarter) << 16) + 256u + cc * 16u, v2);
                    tmem_ld_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 16; j++)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
                } else {
                    tmem_ld_wait();
                }
                if (!to_partial && (a.act != nullptr || a.silu_gather != 0u)) {
                    // gate/up fused: this lane's row is a gate row (even) or the up row of the same output
                    // column (odd).  The gate lane finishes tokens 0-7 of the chunk, the up lane tokens 8-15;
                    // each sends the other the eight values it needs.  The f16 results of the chunk - 16 tokens
                    // x this block's 64 activation columns, from the four warps that share the chunk - meet in
                    // shared memory (the x ring is idle by now) and leave as 16-byte stores, 128 contiguous
                    // bytes per token: full lines for local memory and for the NVLink stores of the gather.
                    const bool is_up = (lane & 1u) != 0u;
                    uint8_t* const tile = smem + slice * 4096u + ((cc >> 2) & 1u) * 2048u;     // two buffers per slice
#pragma unroll
                    for (uint32_t j = 0; j < 8; j++) {
                        const float send = __uint_as_float(is_up ? v[j] : v[8u + j]);
                        const float recv = __shfl_xor_sync(0xFFFFFFFFu, send, 1);
                        const float g = is_up ? recv : __uint_as_float(v[j]);
                        const float u = is_up ? __uint_as_float(v[8u + j]) : recv;
                        const uint32_t tl = is_up ? 8u + j : j;
                        *reinterpret_cast<uint16_t*>(tile + tl * 128u + (16u * quarter + (lane >> 1)) * 2u) =
                            f32_to_f16_bits(silu_mul_f32(g, u));
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(2u + slice) : "memory");
                    const uint32_t i = 32u * quarter + lane, tok = i >> 3, part = i & 7u;
                    const uint32_t t = t0 + tok;
                    if (t < a.m) {
                        const uint4 val = *reinterpret_cast<const uint4*>(tile + tok * 128u + part * 16u);
                        if (a.silu_gather == 0u) {
                            *reinterpret_cast<uint4*>(a.act + (size_t)t * (a.n >> 1) + (n0 >> 1) + part * 8u) = val;
                        } else {
                            const size_t o = (size_t)t * (a.gather_n >> 1) + ((a.gather_n0 + n0) >> 1) + part * 8u;
#pragma unroll
                            for (uint32_t d = 0; d < GATHER_MAX; d++)
                                if (d < a.gather_world) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.gather_y[d]) + o) = val;
                        }
                    }
                } else {
                    // The chunk - 16 tokens x this block's 128 rows, from the four warps that share it - meets in
                    // shared memory (the x ring is idle by now) and leaves as 16-byte stores: a warp writes 512
                    // contiguous bytes of one token where a lane-per-row store would write 128, and the gather's
                    // NVLink stores are full lines.  Two buffers per slice, so one barrier per chunk is enough.
                    float* const tile = reinterpret_cast<float*>(smem + slice * 16384u + ((cc >> 2) & 1u) * 8192u);
#pragma unroll
                    for (uint32_t j = 0; j < 16; j++) tile[j * 128u + 32u * quarter + lane] = __uint_as_float(v[j]);
                    asm volatile("bar.sync %0, 128;" ::"r"(2u + slice) : "memory");
                    const uint32_t i = 32u * quarter + lane;
#pragma unroll
                    for (uint32_t q = 0; q < 4; q++) {
                        const uint32_t p = i + 128u * q, tok = p >> 5, part = p & 31u;
                        const uint32_t t = t0 + tok;
                        if (t < a.m) {
                            float4 val = *reinterpret_cast<const float4*>(tile + tok * 128u + part * 4u);
                            const size_t o = (size_t)t * a.n + n0 + part * 4u;
                            if (res) {
                                const float4 rr = __ldg(reinterpret_cast<const float4*>(res + o));
                                val.x += rr.x; val.y += rr.y; val.z += rr.z; val.w += rr.w;
                            }
                            if (a.gather_world == 0u || to_partial) {
                                *reinterpret_cast<float4*>(out + o) = val;
                            } else {
                                // fused all-gather: the same row segment goes to every GPU's y
                                const size_t og = (size_t)t * a.gather_n + a.gather_n0 + n0 + part * 4u;
#pragma unroll
                                for (uint32_t d = 0; d < GATHER_MAX; d++)
                                    if (d < a.gather_world) *reinterpret_cast<float4*>(a.gather_y[d] + og) = val;
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (TRACE && a.trace && tid == 0) {
        a.trace[16ull * blockIdx.x + 7] = (unsigned long long)clock64();   // epilogue done
        unsigned long long gt;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
        a.trace[16ull * blockIdx.x + 15] = gt;                             // ... in nanoseconds of the GPU's global timer
    }
    cluster_sync_all();          // the partner's shared memory and barriers stay alive until both are done
    if (warp == PAIR_WARP_MMA) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
    }
}

// y = sum over splits of partial[s] (+ r), four floats per thread step; the order of the sum is fixed.
struct GatherDst {
    float* y[GATHER_MAX];
    uint32_t world, n_total, n0, n_local;   // world = 0: plain y
    uint32_t silu;                          // the gathered buffers are f16 [m, n_total/2] of silu(gate) * up
};

// With `act` (or g.silu) set, columns are gate/up interleaved and the kernel writes silu(gate) * up as f16 [m, n/2].
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, uint32_t splits, size_t elems,
                                     const float* __restrict__ r, float* __restrict__ y, const GatherDst g,
                                     uint16_t* __restrict__ act, uint32_t n_local) {
    // launched with programmatic stream serialization behind the GEMM that writes the partials: its
    // blocks are in place when that launch ends
    allow_dependents();
    grid_dependency_wait();
    const size_t n4 = elems / 4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        // the first eight splits' loads are issued together (one trip to L2 instead of one per split); the sum
        // keeps the order of the splits
        float4 v[8];
#pragma unroll
        for (uint32_t s = 0; s < 8u; s++)
            if (s < splits) v[s] = reinterpret_cast<const float4*>(partial + (size_t)s * elems)[i];
        float4 acc = v[0];
#pragma unroll
        for (uint32_t s = 1; s < 8u; s++)
            if (s < splits) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
        for (uint32_t s = 8u; s < splits; s++) {
            const float4 p = reinterpret_cast<const float4*>(partial + (size_t)s * elems)[i];
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        if (r) {
            const float4 q = reinterpret_cast<const float4*>(r)[i];
            acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
        }
        if (act != nullptr || g.silu != 0u) {
            // four columns = two (gate, up) pairs -> two f16 values of row t, columns c/2 and c/2 + 1
            const uint32_t two = (uint32_t)f32_to_f16_bits(silu_mul_f32(acc.x, acc.y)) |
                                 ((uint32_t)f32_to_f16_bits(silu_mul_f32(acc.z, acc.w)) << 16);
            const size_t e = i * 4, t = e / n_local, c = e - t * n_local;
            if (g.world == 0u) {
                reinterpret_cast<uint32_t*>(act)[(t * (n_local >> 1) + (c >> 1)) >> 1] = two;
            } else {
                const size_t o = (t * (g.n_total >> 1) + ((g.n0 + c) >> 1)) >> 1;
#pragma unroll
                for (uint32_t d = 0; d < GATHER_MAX; d++)
                    if (d < g.world) reinterpret_cast<uint32_t*>(g.y[d])[o] = two;
            }
        } else if (g.world == 0u) {
            reinterpret_cast<float4*>(y)[i] = acc;
        } else {
            // fused all-gather: element (t, c) of the local [m, n_local] goes to column n0 + c of every y
            const size_t e = i * 4, t = e / g.n_local, c = e - t * g.n_local;
            const size_t o = t * g.n_total + g.n0 + c;
#pragma unroll
            for (uint32_t d = 0; d < GATHER_MAX; d++)
                if (d < g.world) *reinterpret_cast<float4*>(g.y[d] + o) = acc;
        }
    }
}

}  // namespace lexb
