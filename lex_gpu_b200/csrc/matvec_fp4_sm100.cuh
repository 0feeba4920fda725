// gemm_fp4 for m <= 16 (decode and speculative-verify steps): a split-K matvec that reads the
// packed weights from HBM once.
//
// Same operator as gemm_fp4_sm100.cuh (crates/lex-front/lx/gemm_fp4.lx:16-36): f16 x,
// weights decoded bit-exactly to f16, f32 accumulation.  The reference runs small m
// through different kernels with different arithmetic (crates/lex-msl/src/int8.rs:121-223
// quantises x to int16; crates/lex-front/src/llama.rs:444-499 keeps weights in f32); this
// one keeps gemm_fp4's semantics so one oracle covers every m.
//
// A block owns 16 weight rows at a time and all of K; its 8 warps take K in interleaved slices
// of 128 columns, so the block reads 512 contiguous bytes of each row per round.  Inside a
// slice, lane (g = lane/4, t = lane%4) owns rows g and g+8 and the two groups of 16
// columns 32t..32t+31: one 16-byte load of codes per row, two scale bytes, two decode
// tables per row.  The multiply-accumulate runs on the tensor cores (mma.sync m16n8k16,
// weights as the 16-row operand, up to 8 tokens as the 8-column operand): the integer pipe
// is fully taken by the decode, and the f16 x f16 products are exact in f32 either way.
// Because a contraction may visit K in any order, the 16 K-slots of one mma are mapped to
// 4 columns from each of the 4 lanes' own groups - no weight ever crosses lanes.
//
// Blocks are persistent when x fits in shared memory (the usual case): x is staged once and
// the block walks over row blocks blockIdx.x, +gridDim.x, ...; the loads of the next slice -
// of the next row block at the end - are always in flight while a slice is decoded.
// x in shared memory: each 64-byte run (32 columns, what one lane consumes per slice) is
// stored 72 bytes apart and the token pitch is 32 (mod 128) bytes, which makes the quad's
// four 8-byte reads per token and the eight tokens of a warp hit distinct banks.
#pragma once
#include "sm100_ptx.cuh"
#include "fp4_decode.cuh"

namespace lexb {

constexpr uint32_t MV_ROWS = 16;
constexpr uint32_t MV_WARPS = 8;
constexpr uint32_t MV_THREADS = MV_WARPS * 32;
constexpr uint32_t MV_SLICE = 128;                   // K columns per warp iteration
constexpr uint32_t MV_ROUND = MV_SLICE * MV_WARPS;   // K columns per block round
constexpr uint32_t MV_RED_BYTES = MV_WARPS * MV_ROWS * 16u * 4u;   // one reduction buffer
// The packed weights come through a ring in shared memory filled by asynchronous copies (cp.async): a warp keeps
// MV_DEPTH slices in flight, each lane copying exactly the 2 x 16 bytes of codes it will decode itself (so the ring
// is a per-lane FIFO and its reads are conflict-free) and one lane of each quad the quad's 2 x 8 scale bytes.
// With the loads in registers one slice ahead, the warps spent most of their time waiting for memory.
constexpr uint32_t MV_DEPTH = 3;
constexpr uint32_t MV_STAGE_BYTES = 2u * 512u + 128u;              // codes of row g, codes of row g + 8, scale bytes
constexpr uint32_t MV_RING_BYTES = MV_WARPS * MV_DEPTH * MV_STAGE_BYTES;

struct MatvecArgs {
    const __half* x;      // [m, k]
    const uint8_t* wq;    // [n, k/2]
    const uint8_t* ws;    // [n, k/16]
    const float* wg;      // [n]
    const float* r;       // [m, n] or null
    float* y;             // [m, n]
    uint32_t m, n, k;
    uint32_t kc;          // K columns of x staged per chunk: multiple of MV_ROUND
};

// token pitch in bytes: kc/32 runs of 72 bytes, padded to 32 (mod 128)
__host__ __device__ constexpr uint32_t matvec_x_pitch(uint32_t kc) {
    return (kc / 32u) * 72u + ((32u + 128u - ((kc / 32u) * 72u) % 128u) % 128u);
}
// two reduction buffers (alternating per row block), the ring (when used), then the x chunk
__host__ __device__ constexpr uint32_t matvec_smem_bytes(uint32_t m, uint32_t kc, bool ring) {
    return 2u * MV_RED_BYTES + (ring ? MV_RING_BYTES : 0u) + 128u + m * matvec_x_pitch(kc) + 16u;   // 128 bytes of zeros before x
}
// The ring pays while x leaves room for several blocks per SM: up to 4 tokens.  Beyond, the staged x fills shared
// memory and the ring would cost a resident block; the weights then come through registers, one slice ahead.
__host__ __device__ constexpr bool matvec_uses_ring(uint32_t m) { return m <= 4u; }

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MvLoad {
    uint4 qa, qb;        // 32 codes of row g / row g+8
    uint32_t sa, sb;     // their two scale bytes (low 16 bits)
};

// 16, 8 or 0 bytes from global to shared memory without passing through registers; src_bytes = 0 fills with zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <uint32_t N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// HI: m > 8, a second group of 8 tokens; RAGGED: k % 128 != 0; RING: packed weights through the cp.async ring
template <bool HI, bool RAGGED, bool RING>
__global__ void __launch_bounds__(MV_THREADS) matvec_fp4_kernel(const MatvecArgs a) {
    extern __shared__ __align__(16) uint8_t mv_smem[];
    float* const red = reinterpret_cast<float*>(mv_smem);               // [2][warp][row 16][token 16]
    uint8_t* const ring = mv_smem + 2u * MV_RED_BYTES;                  // [warp][MV_DEPTH] stages of packed weights
    uint8_t* const zeros = ring + (RING ? MV_RING_BYTES : 0u);          // 128 bytes: x of a token that does not exist
    uint8_t* const xs = zeros + 128u;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    // launched with programmatic stream serialization: the blocks are in place when the launch ahead ends
    allow_dependents();
    grid_dependency_wait();
    const uint32_t k = a.k, kc = a.kc;
    const uint32_t pitch = matvec_x_pitch(kc);
    const uint32_t slices = (k + MV_SLICE - 1u) / MV_SLICE;             // per row block
    const uint32_t row_blocks = a.n / MV_ROWS;
    const bool resident = kc >= k;                                      // all of x staged once
    constexpr bool lane_in_k_always = !RAGGED;

    // lanes whose token does not exist (and lanes past the end of K) read the zero block instead
    const bool have_lo = g < a.m, have_hi = HI && (g + 8u) < a.m;

    // x[:, k0:k1] -> shared memory, 8 bytes at a time (coalesced in, conflict-free out)
    auto stage_x = [&](uint32_t k0, uint32_t k1) {
        const uint32_t units = (k1 - k0) / 4u;                          // 8-byte units per token
        for (uint32_t idx = tid; idx < a.m * units; idx += MV_THREADS) {
            const uint32_t tok = idx / units, u = idx - tok * units;
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(a.x + (size_t)tok * k + k0) + u);
            *reinterpret_cast<uint2*>(xs + tok * pitch + (u >> 3) * 72u + (u & 7u) * 8u) = v;
        }
        if (tid < 16u) *reinterpret_cast<uint2*>(zeros + tid * 8u) = make_uint2(0u, 0u);
    };

    // This warp's ring.  Stage layout: [codes of row g: 32 lanes x 16 B][codes of row g + 8][scales: 16 rows x 8 B].
    uint8_t* const my_ring = ring + warp * (MV_DEPTH * MV_STAGE_BYTES);
    const uint32_t my_ring_u32 = smem_u32(my_ring);
    const size_t q_pitch8 = (size_t)8u * (k / 2), s_pitch8 = (size_t)8u * (k / 16);
    // asynchronous copies of slice `it` of row block `rb` into stage `st` (one commit group, also when the slice
    // does not exist: the groups are counted)
    auto issue = [&](uint32_t rb, uint32_t it, uint32_t st, bool exists) {
        if (exists) {
            const uint32_t col = it * MV_SLICE + 32u * t;               // first of this lane's 32 columns
            const uint32_t in_k = (lane_in_k_always || col < k) ? 1u : 0u;   // k % 32 == 0: all 32 or none (then zeros)
            const uint32_t colc = in_k ? col : 0u;
            const uint8_t* qa_p = a.wq + (size_t)(rb * MV_ROWS + g) * (k / 2) + colc / 2u;
            const uint32_t dst = my_ring_u32 + st * MV_STAGE_BYTES + lane * 16u;
            cp_async_16(dst, qa_p, 16u * in_k);
            cp_async_16(dst + 512u, qa_p + q_pitch8, 16u * in_k);
            if (RAGGED) {
                // k % 128 != 0: a row's scale bytes are not 8-byte aligned, so each lane fetches its own two
                // (plain loads; these shapes are small)
                const uint8_t* sa_p = a.ws + (size_t)(rb * MV_ROWS + g) * (k / 16) + colc / 16u;
                uint8_t* sdst = my_ring + st * MV_STAGE_BYTES + 1024u + g * 8u + 2u * t;
                *reinterpret_cast<unsigned short*>(sdst) = in_k ? __ldg(reinterpret_cast<const unsigned short*>(sa_p)) : (unsigned short)0;
                *reinterpret_cast<unsigned short*>(sdst + 64u) =
                    in_k ? __ldg(reinterpret_cast<const unsigned short*>(sa_p + s_pitch8)) : (unsigned short)0;
            } else if (t == 0u) {
                // the quad's scale bytes: columns it * 128 .. +127 of rows g and g + 8, 8 bytes each
                const uint8_t* sa_p = a.ws + (size_t)(rb * MV_ROWS + g) * (k / 16) + it * (MV_SLICE / 16u);
                const uint32_t sdst = my_ring_u32 + st * MV_STAGE_BYTES + 1024u + g * 8u;
                cp_async_8(sdst, sa_p, 8u);
                cp_async_8(sdst + 64u, sa_p + s_pitch8, 8u);
            }
        }
        cp_async_commit();
    };
    // the register path (RING = false): this lane's loads for slice `it` of row block `rb`
    auto load = [&](uint32_t rb, uint32_t it) {
        MvLoad L;
        const uint32_t col = it * MV_SLICE + 32u * t;
        if (lane_in_k_always || col < k) {
            const uint8_t* qa_p = a.wq + (size_t)(rb * MV_ROWS + g) * (k / 2) + col / 2u;
            const uint8_t* sa_p = a.ws + (size_t)(rb * MV_ROWS + g) * (k / 16) + col / 16u;
            L.qa = __ldg(reinterpret_cast<const uint4*>(qa_p));
            L.qb = __ldg(reinterpret_cast<const uint4*>(qa_p + q_pitch8));
            L.sa = __ldg(reinterpret_cast<const unsigned short*>(sa_p));
            L.sb = __ldg(reinterpret_cast<const unsigned short*>(sa_p + s_pitch8));
        } else {                                                        // past the end: zero codes (their lane multiplies by 1.0)
            L.qa = make_uint4(0, 0, 0, 0);
            L.qb = make_uint4(0, 0, 0, 0);
            L.sa = 0u;
            L.sb = 0u;
        }
        return L;
    };
    auto take = [&](uint32_t st) {
        MvLoad L;
        const uint8_t* sp = my_ring + st * MV_STAGE_BYTES;
        L.qa = *reinterpret_cast<const uint4*>(sp + lane * 16u);
        L.qb = *reinterpret_cast<const uint4*>(sp + 512u + lane * 16u);
        L.sa = *reinterpret_cast<const unsigned short*>(sp + 1024u + g * 8u + 2u * t);
        L.sb = *reinterpret_cast<const unsigned short*>(sp + 1024u + 64u + g * 8u + 2u * t);
        return L;
    };

    // (started before x is staged: the first slices land meanwhile)
    // the copy cursor runs MV_DEPTH slices ahead of the decode, in the same order: this warp's slices of a row
    // block, then those of the block's next row block
    uint32_t rb_c = blockIdx.x, it_c = warp, st_c = 0;
    auto issue_next = [&]() {
        while (rb_c < row_blocks && it_c >= slices) {                   // (a warp with no slice in this row block)
            it_c = warp;
            rb_c += gridDim.x;
        }
        const bool exists = rb_c < row_blocks && it_c < slices;
        issue(rb_c, it_c, st_c, exists);
        st_c = st_c + 1u == MV_DEPTH ? 0u : st_c + 1u;
        if (exists) {
            it_c += MV_WARPS;
            if (it_c >= slices) {
                it_c = warp;
                rb_c += gridDim.x;
            }
        }
    };
    MvLoad nxt{};
    if constexpr (RING) {
#pragma unroll
        for (uint32_t d = 0; d < MV_DEPTH; d++) issue_next();
    } else {
        nxt = load(blockIdx.x < row_blocks ? blockIdx.x : 0u, warp < slices ? warp : 0u);
    }

    if (resident) {
        stage_x(0, k);
        __syncthreads();
    }

    uint32_t rb = blockIdx.x;
    uint32_t it = warp;
    uint32_t st = 0;
    uint32_t parity = 0;

    for (; rb < row_blocks; rb += gridDim.x, parity ^= 1u) {
        const uint32_t n0 = rb * MV_ROWS;
        const float ga = __ldg(a.wg + n0 + g), gb = __ldg(a.wg + n0 + g + 8u);
        float c_lo[4] = {0.f, 0.f, 0.f, 0.f};
        float c_hi[4] = {0.f, 0.f, 0.f, 0.f};

        for (uint32_t k0 = 0; k0 < k; k0 += kc) {
            const uint32_t k1 = (k0 + kc < k) ? (k0 + kc) : k;
            if (!resident) {
                __syncthreads();                                        // previous chunk fully consumed
                stage_x(k0, k1);
                __syncthreads();
            }
            while (it < slices && it * MV_SLICE < k1) {
                MvLoad cur;
                if constexpr (RING) {
                    cp_async_wait<MV_DEPTH - 1>();                      // the oldest slice in flight has landed
                    __syncwarp();                                       // (the scale bytes were copied by lane 0 of the quad)
                    cur = take(st);
                    __syncwarp();                                       // every lane has read the stage: refill it
                    issue_next();
                    st = st + 1u == MV_DEPTH ? 0u : st + 1u;
                } else {
                    cur = nxt;
                    // next slice of this row block, or the first slice of the block's next row block
                    uint32_t it_n = it + MV_WARPS, rb_n = rb;
                    if (it_n >= slices) {
                        it_n = warp;
                        rb_n = rb + gridDim.x;
                    }
                    if (rb_n < row_blocks && it_n < slices) nxt = load(rb_n, it_n);
                }
                const bool in_range = lane_in_k_always || (it * MV_SLICE + 32u * t < k);
                // a lane past the end of K multiplies zero codes by 1.0, never by a row scale
                // that might be infinite
                const float ga_e = in_range ? ga : 1.0f, gb_e = in_range ? gb : 1.0f;
                // this lane's 64 bytes of x per token: run (slice offset / 32 + t), 72 bytes apart
                const uint32_t xoff = (((it * MV_SLICE - k0) >> 5) + t) * 72u;
                const uint8_t* x_lo = (have_lo && in_range) ? xs + g * pitch + xoff : zeros;
                const uint8_t* x_hi = (have_hi && in_range) ? xs + (g + 8u) * pitch + xoff : zeros;
                const float2 sca = e4m3x2_to_f32(cur.sa), scb = e4m3x2_to_f32(cur.sb);

#pragma unroll
                for (uint32_t grp = 0; grp < 2; grp++) {
                    const GroupTable ta = make_group_table_f32(grp ? sca.y : sca.x, ga_e);
                    const GroupTable tb = make_group_table_f32(grp ? scb.y : scb.x, gb_e);
#pragma unroll
                    for (uint32_t wd = 0; wd < 2; wd++) {
                        const uint32_t wa = grp ? (wd ? cur.qa.w : cur.qa.z) : (wd ? cur.qa.y : cur.qa.x);
                        const uint32_t wb = grp ? (wd ? cur.qb.w : cur.qb.z) : (wd ? cur.qb.y : cur.qb.x);
                        uint32_t oa[4], ob[4];
                        decode8(ta, wa, oa[0], oa[1], oa[2], oa[3]);
                        decode8(tb, wb, ob[0], ob[1], ob[2], ob[3]);
#pragma unroll
                        for (uint32_t hf = 0; hf < 2; hf++) {
                            const uint32_t unit = 4u * grp + 2u * wd + hf;   // 8-byte unit of the lane's 64 bytes
                            const uint2 bl = *reinterpret_cast<const uint2*>(x_lo + 8u * unit);
                            mma_m16n8k16(c_lo, oa[2 * hf], ob[2 * hf], oa[2 * hf + 1], ob[2 * hf + 1], bl.x, bl.y);
                            if (HI) {
                                const uint2 bh = *reinterpret_cast<const uint2*>(x_hi + 8u * unit);
                                mma_m16n8k16(c_hi, oa[2 * hf], ob[2 * hf], oa[2 * hf + 1], ob[2 * hf + 1], bh.x, bh.y);
                            }
                        }
                    }
                }
                it += MV_WARPS;
            }
        }
        it = warp;                                                      // first slice of the next row block

        // cross-warp reduction in a fixed order, then one coalesced store per token.  Two buffers
        // alternate, so one barrier per row block is enough.
        float* const rw = red + parity * (MV_WARPS * MV_ROWS * 16u) + warp * (MV_ROWS * 16u);
        rw[g * 16u + 2u * t] = c_lo[0];
        rw[g * 16u + 2u * t + 1u] = c_lo[1];
        rw[(g + 8u) * 16u + 2u * t] = c_lo[2];
        rw[(g + 8u) * 16u + 2u * t + 1u] = c_lo[3];
        if (HI) {
            rw[g * 16u + 8u + 2u * t] = c_hi[0];
            rw[g * 16u + 8u + 2u * t + 1u] = c_hi[1];
            rw[(g + 8u) * 16u + 8u + 2u * t] = c_hi[2];
            rw[(g + 8u) * 16u + 8u + 2u * t + 1u] = c_hi[3];
        }
        __syncthreads();
        if (tid < MV_ROWS * a.m) {
            const uint32_t row = tid & 15u, tok = tid >> 4;
            const float* rp = red + parity * (MV_WARPS * MV_ROWS * 16u) + row * 16u + tok;
            float s = 0.f;
#pragma unroll
            for (uint32_t w = 0; w < MV_WARPS; w++) s += rp[w * (MV_ROWS * 16u)];
            const size_t o = (size_t)tok * a.n + n0 + row;
            if (a.r) s = s + __ldg(a.r + o);
            a.y[o] = s;
        }
    }
}

}  // namespace lexb
