// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA tile
// loads, tcgen05 (TMEM allocation, MMA issue, commit, TMEM loads) and proxy fences.
// Every wait is bounded: it gives up after a fixed number of clock cycles and reports
// failure so that the caller can record a status code and leave the kernel in order.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace lexb {

// Position in a ring of `depth` stages: stage index and phase bit, advanced without the integer
// division that `k % depth`, `(k / depth) & 1` would cost on every K step of a single-warp role.
struct RingPos {
    uint32_t s = 0, ph = 0;
    __device__ __forceinline__ void advance(uint32_t depth) {
        if (++s == depth) {
            s = 0;
            ph ^= 1u;
        }
    }
    // n steps at once (n small: a few turns of the loop at most)
    __device__ __forceinline__ void advance_by(uint32_t n, uint32_t depth) {
        s += n;
        while (s >= depth) {
            s -= depth;
            ph ^= 1u;
        }
    }
    // position of item `index` (divides: for the start of a loop, not for its body)
    __device__ __forceinline__ void seek(uint32_t index, uint32_t depth) {
        s = index % depth;
        ph = (index / depth) & 1u;
    }
};

// Status codes a kernel may OR into the status word (0 = clean run).
enum : uint32_t {
    ST_WAIT_X_FULL = 1u << 0,      // MMA thread gave up waiting for a TMA x tile
    ST_WAIT_W_FULL = 1u << 1,      // MMA thread gave up waiting for the dequantised W tile
    ST_WAIT_EMPTY_TMA = 1u << 2,   // TMA producer gave up waiting for a free stage
    ST_WAIT_EMPTY_DEQ = 1u << 3,   // dequant thread gave up waiting for a free stage
    ST_WAIT_ACC = 1u << 4,         // epilogue gave up waiting for the accumulator
    ST_WAIT_DRAIN = 1u << 5,       // producer gave up waiting for its own copies in flight
    ST_BAD_ARGS = 1u << 8,         // a device-side argument check failed
    ST_WAIT_NEVER = 1u << 16,      // the self-test wait ran out, as it is meant to
};

constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;   // about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same test with a suspend-time hint: the hardware may park the thread until the phase completes or
// `hint_ns` nanoseconds pass, instead of returning at once.  A warp that waits this way does not poll: it
// takes no issue slots and no shared-memory cycles from the warps that are working.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
constexpr uint32_t WAIT_PARK_NS = 4000;      // one parked attempt; the loop around it keeps the overall bound
// Bounded wait.  `abort_flag` (shared memory) lets one role's failure end the others' waits early.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait_parked(bar, parity, WAIT_PARK_NS)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
    return true;
}

// One lane of a fully converged warp (the same one every time).  The role loops run on the whole
// warp with warp-uniform values and only the asynchronous instruction itself is issued by the elected
// lane: that lets the compiler keep addresses and descriptors in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization
// attribute may start before the kernel ahead of it in the stream has finished; it must not touch
// global memory that kernel may still write (or that it still reads and this one overwrites) before
// grid_dependency_wait() returns.  allow_dependents() lets the next such kernel be scheduled as soon as
// resources free up.  Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 2-D tiled TMA load global -> shared, completion counted in bytes on an mbarrier.
// c0 is the innermost coordinate: c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, bytes a multiple of 16), completion
// counted on an mbarrier like a tile load.
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// The same box into L2 only: a hint, nothing waits for it.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {   // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile in the 128-byte-swizzled layout:
// rows of 64 f16 (128 bytes), 8-row groups 1024 bytes apart, the 16-byte chunks of a row
// XORed with (row & 7).  The tile base must be 1024-byte aligned; stepping K by 16
// elements inside the 128-byte row is +32 bytes on the start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
    d |= 1ull << 16;                                           // leading byte offset (unused with swizzle), bits [16,30)
    d |= static_cast<uint64_t>(1024u >> 4) << 32;              // stride byte offset: 8 rows x 128 B, bits [32,46)
    d |= 1ull << 46;                                           // descriptor version for sm_100
    d |= 2ull << 61;                                           // layout type: SWIZZLE_128B
    return d;
}

// The single thread that issues the MMAs shares its scheduler with decode warps, so every
// instruction it spends between two MMAs delays the tensor pipe.  These helpers keep that count
// small: the high half of a descriptor is constant, the low half is (address >> 4) | LBO, and
// stepping K by 16 is +2 on the low half.
constexpr uint32_t UMMA_DESC_HI_SW128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) {
    return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}
#define LEXB_UMMA_ASM(GROUP, COLLECTOR, PRED_SETUP)                                                          \
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t" PRED_SETUP                                  \
                 "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"                                        \
                 "tcgen05.mma.cta_group::" GROUP ".kind::f16" COLLECTOR " [%0], da, db, %3, p;\n\t}"          \
                 ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(UMMA_DESC_HI_SW128), "r"(accumulate)   \
                 : "memory")
// accumulate is a run-time flag
__device__ __forceinline__ void umma1_flag(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    LEXB_UMMA_ASM("1", "", "setp.ne.b32 p, %5, 0;\n\t");
}
__device__ __forceinline__ void umma2_flag(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    LEXB_UMMA_ASM("2", "", "setp.ne.b32 p, %5, 0;\n\t");
}
__device__ __forceinline__ void umma2_flag_fill(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    LEXB_UMMA_ASM("2", ".collector::a::fill", "setp.ne.b32 p, %5, 0;\n\t");
}
__device__ __forceinline__ void umma2_flag_lastuse(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    LEXB_UMMA_ASM("2", ".collector::a::lastuse", "setp.ne.b32 p, %5, 0;\n\t");
}
// accumulate always
__device__ __forceinline__ void umma1_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    const uint32_t accumulate = 1;
    LEXB_UMMA_ASM("1", "", "setp.eq.b32 p, 0, 0;\n\t");
}
__device__ __forceinline__ void umma2_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    const uint32_t accumulate = 1;
    LEXB_UMMA_ASM("2", "", "setp.eq.b32 p, 0, 0;\n\t");
}
__device__ __forceinline__ void umma2_acc_fill(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    const uint32_t accumulate = 1;
    LEXB_UMMA_ASM("2", ".collector::a::fill", "setp.eq.b32 p, 0, 0;\n\t");
}
__device__ __forceinline__ void umma2_acc_lastuse(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    const uint32_t accumulate = 1;
    LEXB_UMMA_ASM("2", ".collector::a::lastuse", "setp.eq.b32 p, 0, 0;\n\t");
}

// A operand from tensor memory (rows = lanes, two f16 of K per 32-bit column; written by tcgen05.st), B from shared
// memory: nothing of the A tile crosses the shared-memory pipe.  `a_tmem` is the tile's address at lane 0; stepping
// K by 16 elements is +8 columns.
__device__ __forceinline__ void umma2_ts_flag(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "mov.b64 db, {%2, %4};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(UMMA_DESC_HI_SW128), "r"(accumulate)
                 : "memory");
}
// Each lane of the warp writes 32 consecutive 32-bit columns of its own TMEM lane (the warp's lane quarter).
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Instruction descriptor, kind::f16: f16 x f16 -> f32, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(uint32_t M, uint32_t N) {
    return (1u << 4)              // D format f32
           | (0u << 7)            // A format f16
           | (0u << 10)           // B format f16
           | (0u << 15) | (0u << 16)   // A, B K-major
           | ((N >> 3) << 17) | ((M >> 4) << 24);
}


// ---- block-scaled FP4 MMA (kind::mxf4nvf4): E2M1 operands, one UE4M3 scale per 16 values of K ----
// Both operands are packed E2M1 (two per byte, even K in the low nibble), K-major in the same
// 128-byte-swizzled layout as above (a 128-byte row is 256 values of K); one instruction covers
// K = 64 (32 bytes: +2 on the low descriptor half).  The scales of the 128 rows of A (and of the N
// rows of B) for one instruction sit in tensor memory: lane (row % 32) of every 32-lane quarter,
// byte 4 * (row / 32) + (group of 16 within the 64), i.e. four 32-bit columns per instruction.
__host__ __device__ constexpr uint32_t umma_idesc_mxf4nvf4(uint32_t M, uint32_t N) {
    return (1u << 7)              // A format E2M1
           | (1u << 10)           // B format E2M1
           | (0u << 15) | (0u << 16)   // A, B K-major
           | ((N >> 3) << 17)
           | (0u << 23)           // scale format UE4M3
           | ((M >> 4) << 24);    // scale-factor ids (bits 4-5, 29-30) 0: all four bytes of a column are used
}
__device__ __forceinline__ void umma1_mxf4nvf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %7, 0;\n\t"
        "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(UMMA_DESC_HI_SW128), "r"(sfa_tmem), "r"(sfb_tmem),
          "r"(accumulate)
        : "memory");
}
// Descriptor of a 512-byte scale block in shared memory: 32 rows of 16 bytes, contiguous (no swizzle;
// 8-row core matrices 128 bytes apart).
__device__ __forceinline__ uint64_t umma_desc_scale_block(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= 1ull << 16;                                  // leading byte offset: one 16-byte column only
    d |= static_cast<uint64_t>(128u >> 4) << 32;      // stride byte offset between 8-row groups
    d |= 1ull << 46;
    return d;
}
// Shared memory -> tensor memory: 32 rows x 16 bytes into lanes 0-31, columns [c, c + 4), repeated in
// all four 32-lane quarters.  Asynchronous; ordered with the MMAs the same thread issues after it, and
// tracked by that thread's next commit.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}

}  // namespace lexb

// ---- two-CTA (cta_group::2) variants: a pair of CTAs in one cluster shares each MMA ------
namespace lexb {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs: nobody passes until everybody has arrived.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The shared::cluster address of `local_addr` as seen in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Arrivals on a barrier of the partner CTA use the default (CTA-scope) release, as CUTLASS's two-SM
// kernels do: a cluster-scope release costs a fence of about a thousand cycles per call, which on a
// once-per-K-step path set the pace of the whole main loop.  What the partner's barrier guards (its
// W tile, written and proxy-fenced in its own shared memory before this arrive) is read by the tensor
// core of that same SM.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
                 "r"(bytes)
                 : "memory");
}
// TMA tile load of a CTA pair: the data lands in this CTA's shared memory, the byte count is
// reported to the barrier at `bar_cluster_addr`, which may live in the partner CTA.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {   // one warp in each CTA
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One MMA over the pair: M = 256 (128 rows of A from each CTA), N up to 256 (half of B from each).
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask`, once the
// MMAs issued so far have finished.  (A barrier signal, not a data copy.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}

}  // namespace lexb
