// gemm_fp4 for m <= 16 (decode and speculative-verify steps): a split-K matvec that is
// bound by reading the packed weights from HBM once.
//
// Same operator as gemm_fp4_sm100.cuh (crates/lex-front/lx/gemm_fp4.lx:16-36): f16 x,
// weights decoded bit-exactly to f16, f32 accumulation.  The reference runs small m
// through different kernels with different arithmetic (crates/lex-msl/src/int8.rs:121-223
// quantises x to int16; crates/lex-front/src/llama.rs:444-499 keeps weights in f32); this
// one keeps gemm_fp4's semantics so one oracle covers every m.
//
// One CTA owns 16 weight rows and all of K; its 8 warps take K in interleaved slices of
// 128 columns, so the CTA reads 512 contiguous bytes of each row per round.  Inside a
// slice, lane (g = lane/4, t = lane%4) owns rows g and g+8 and the two groups of 16
// columns 32t..32t+31: one 16-byte load of codes per row, two scale bytes, two decode
// tables per row.  The multiply-accumulate runs on the tensor cores (mma.sync m16n8k16,
// weights as the 16-row operand, up to 8 tokens as the 8-column operand): the CUDA cores
// are fully taken by the decode, and the f16 x f16 products are exact in f32 either way.
// Because a contraction may visit K in any order, the 16 K-slots of one mma are mapped to
// 4 columns from each of the 4 lanes' own groups - no weight ever crosses lanes.
// x is staged in shared memory (chunks of K when m * k is large) and read conflict-free.
#pragma once
#include "fp4_decode.cuh"

namespace lexb {

constexpr uint32_t MV_ROWS = 16;
constexpr uint32_t MV_WARPS = 8;
constexpr uint32_t MV_THREADS = MV_WARPS * 32;
constexpr uint32_t MV_SLICE = 128;                   // K columns per warp iteration
constexpr uint32_t MV_ROUND = MV_SLICE * MV_WARPS;   // K columns per CTA round

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

// bytes of shared memory: x chunk (pitch 2*kc + 8 bytes per token) or the reduction scratch
__host__ __device__ constexpr uint32_t matvec_smem_bytes(uint32_t m, uint32_t kc) {
    const uint32_t xb = m * (2u * kc + 8u);
    const uint32_t rb = MV_WARPS * MV_ROWS * 16u * 4u;
    return (xb > rb ? xb : rb) + 16u;
}

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

template <bool HI>   // HI: m > 8, a second group of 8 tokens
__global__ void __launch_bounds__(MV_THREADS) matvec_fp4_kernel(const MatvecArgs a) {
    extern __shared__ __align__(16) uint8_t mv_smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t n0 = blockIdx.x * MV_ROWS;
    const uint32_t row_a = n0 + g, row_b = n0 + g + 8u;
    const uint32_t k = a.k, kc = a.kc;
    const uint32_t pitch = 2u * kc + 8u;             // bytes; = 8 (mod 128): conflict-free 8-byte reads
    const uint32_t total_it = (k + MV_SLICE - 1u) / MV_SLICE;

    const float ga = __ldg(a.wg + row_a), gb = __ldg(a.wg + row_b);
    const uint8_t* qa_row = a.wq + (size_t)row_a * (k / 2) + 16u * t;
    const uint8_t* qb_row = a.wq + (size_t)row_b * (k / 2) + 16u * t;
    const uint8_t* sa_row = a.ws + (size_t)row_a * (k / 16) + 2u * t;
    const uint8_t* sb_row = a.ws + (size_t)row_b * (k / 16) + 2u * t;
    // Lanes with t >= 2 take their two groups in the other order, so that the four lanes of
    // a quad read x at 0, 64, 32 and 96 (mod 128) bytes: distinct banks.
    const bool swap = (t & 2u) != 0u;

    auto load = [&](uint32_t it) {
        MvLoad L;
        const uint32_t col = it * MV_SLICE + 32u * t;         // first column of this lane's 32
        if (col < k) {                                         // k % 32 == 0: all 32 or none
            L.qa = __ldg(reinterpret_cast<const uint4*>(qa_row + (size_t)it * (MV_SLICE / 2)));
            L.qb = __ldg(reinterpret_cast<const uint4*>(qb_row + (size_t)it * (MV_SLICE / 2)));
            L.sa = __ldg(reinterpret_cast<const unsigned short*>(sa_row + (size_t)it * (MV_SLICE / 16)));
            L.sb = __ldg(reinterpret_cast<const unsigned short*>(sb_row + (size_t)it * (MV_SLICE / 16)));
        } else {                                               // past the end: zero codes, unit scale
            L.qa = make_uint4(0, 0, 0, 0);
            L.qb = make_uint4(0, 0, 0, 0);
            L.sa = 0x3838u;
            L.sb = 0x3838u;
        }
        return L;
    };

    float c_lo[4] = {0.f, 0.f, 0.f, 0.f};
    float c_hi[4] = {0.f, 0.f, 0.f, 0.f};

    uint32_t it = warp;
    MvLoad nxt = load(it < total_it ? it : 0u);

    const uint32_t tok_lo = g, tok_hi = g + 8u;
    const bool have_lo = tok_lo < a.m, have_hi = HI && tok_hi < a.m;

    for (uint32_t k0 = 0; k0 < k; k0 += kc) {
        const uint32_t k1 = (k0 + kc < k) ? (k0 + kc) : k;
        __syncthreads();                                       // previous chunk fully consumed
        {   // stage x[:, k0:k1] as f16, 8 bytes at a time (coalesced in, conflict-free out)
            const uint32_t units = (k1 - k0) / 4u;             // 8-byte units per token
            for (uint32_t idx = tid; idx < a.m * units; idx += MV_THREADS) {
                const uint32_t tok = idx / units, u = idx - tok * units;
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(a.x + (size_t)tok * k + k0) + u);
                *reinterpret_cast<uint2*>(mv_smem + tok * pitch + 8u * u) = v;
            }
        }
        __syncthreads();
        while (it < total_it && it * MV_SLICE < k1) {
            const MvLoad cur = nxt;
            const uint32_t it_next = it + MV_WARPS;
            if (it_next < total_it) nxt = load(it_next);

            // this lane's 64 bytes of x per token start here; groups swapped for t >= 2
            const uint32_t xoff = (it * MV_SLICE - k0 + 32u * t) * 2u;
            const uint8_t* x_lo = mv_smem + tok_lo * pitch + xoff;
            const uint8_t* x_hi = mv_smem + tok_hi * pitch + xoff;
            const bool in_range = it * MV_SLICE + 32u * t < k;
            // a lane past the end of K multiplies zero codes by 1.0, never by a row scale
            // that might be infinite
            const float ga_e = in_range ? ga : 1.0f, gb_e = in_range ? gb : 1.0f;

#pragma unroll
            for (uint32_t grp = 0; grp < 2; grp++) {
                const uint32_t ag = swap ? (grp ^ 1u) : grp;              // actual group of this step
                uint32_t wa0, wa1, wb0, wb1, sca, scb;
                if (ag == 0) { wa0 = cur.qa.x; wa1 = cur.qa.y; wb0 = cur.qb.x; wb1 = cur.qb.y; sca = cur.sa & 0xFFu; scb = cur.sb & 0xFFu; }
                else         { wa0 = cur.qa.z; wa1 = cur.qa.w; wb0 = cur.qb.z; wb1 = cur.qb.w; sca = (cur.sa >> 8) & 0xFFu; scb = (cur.sb >> 8) & 0xFFu; }
                const GroupTable ta = make_group_table(sca, ga_e);
                const GroupTable tb = make_group_table(scb, gb_e);
#pragma unroll
                for (uint32_t wd = 0; wd < 2; wd++) {
                    uint32_t oa[4], ob[4];
                    decode8(ta, wd ? wa1 : wa0, oa[0], oa[1], oa[2], oa[3]);
                    decode8(tb, wd ? wb1 : wb0, ob[0], ob[1], ob[2], ob[3]);
#pragma unroll
                    for (uint32_t hf = 0; hf < 2; hf++) {
                        const uint32_t unit = 4u * ag + 2u * wd + hf;      // 8-byte unit of this lane's 64 B of x
                        uint2 bl = make_uint2(0u, 0u);
                        if (have_lo && in_range) bl = *reinterpret_cast<const uint2*>(x_lo + 8u * unit);
                        mma_m16n8k16(c_lo, oa[2 * hf], ob[2 * hf], oa[2 * hf + 1], ob[2 * hf + 1], bl.x, bl.y);
                        if (HI) {
                            uint2 bh = make_uint2(0u, 0u);
                            if (have_hi && in_range) bh = *reinterpret_cast<const uint2*>(x_hi + 8u * unit);
                            mma_m16n8k16(c_hi, oa[2 * hf], ob[2 * hf], oa[2 * hf + 1], ob[2 * hf + 1], bh.x, bh.y);
                        }
                    }
                }
            }
            it = it_next;
        }
    }

    // cross-warp reduction in a fixed order, then one coalesced store per token
    __syncthreads();
    float* red = reinterpret_cast<float*>(mv_smem);            // [warp][row 16][token 16]
    {
        float* rw = red + warp * (MV_ROWS * 16u);
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
    }
    __syncthreads();
    if (tid < MV_ROWS * a.m) {
        const uint32_t row = tid & 15u, tok = tid >> 4;
        float s = 0.f;
#pragma unroll
        for (uint32_t w = 0; w < MV_WARPS; w++) s += red[w * (MV_ROWS * 16u) + row * 16u + tok];
        const size_t o = (size_t)tok * a.n + n0 + row;
        if (a.r) s = s + __ldg(a.r + o);
        a.y[o] = s;
    }
}

}  // namespace lexb
