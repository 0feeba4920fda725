// Bit-exact NVFP4 decode for sm_100a: E2M1 code x E4M3 group scale x f32 row scale -> f16.
//
// The value every kernel in this library multiplies by is the one lex's reference
// interpreter stages (crates/lex-front/src/interp.rs:643-657, then :500-507):
//
//     w32 = fl32( fl32( e2m1(code) * e4m3(scale) ) * wg[row] )     left to right
//     w16 = round_to_nearest_even_f16( w32 )
//
// The first product is exact (at most 6 significant bits), so only the multiply by
// the row scale and the conversion round.  The reference's own GPU kernels fold the
// group scale into the row scale first (crates/lex-msl/src/gemm.rs:254-255,
// crates/lex-msl/src/dialect.rs:768-791), which rounds differently in about one
// weight in 10^5 and turns the NaN scale bytes into +-480; this file follows the
// interpreter instead.
//
// Method: a group of 16 weights shares its scale, so it has only 8 distinct
// magnitudes.  They are computed once per group (16 f32 multiplies, 4 packed
// f32->f16x2 conversions) and kept as a register table split into a low-byte plane
// and a high-byte plane; each weight is then one byte-permute lookup per plane,
// selected by its 3 magnitude bits, and the sign bit of the code is XORed in.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace lexb {

// Two OCP e4m3fn bytes -> two f32, exact for all 256 byte values: the hardware conversion to f16 is
// exact (every E4M3 value, subnormals included, is an f16 value) and maps the two NaN bytes
// (exponent 15, mantissa 7; interp.rs:41-42) to NaN; f16 -> f32 is exact as well.
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t two_bytes) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<unsigned short>(two_bytes)));
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) { return e4m3x2_to_f32(b & 0xFFu).x; }

__device__ __forceinline__ uint32_t pack_f16x2_rn(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// The 8 magnitudes of one group as f16, split into byte planes:
// lo.x/lo.y hold the low bytes of entries 0-3 / 4-7, hi.x/hi.y the high bytes.
struct GroupTable {
    uint32_t lo0, lo1, hi0, hi1;
};

__device__ __forceinline__ GroupTable make_group_table_f32(float s, float wg) {
    // (e2m1 * s) is exact; __fmul_rn keeps the compiler from reassociating or contracting.
    const float p0 = __fmul_rn(__fmul_rn(0.0f, s), wg);
    const float p1 = __fmul_rn(__fmul_rn(0.5f, s), wg);
    const float p2 = __fmul_rn(s, wg);
    const float p3 = __fmul_rn(__fmul_rn(1.5f, s), wg);
    const float p4 = __fmul_rn(__fmul_rn(2.0f, s), wg);
    const float p5 = __fmul_rn(__fmul_rn(3.0f, s), wg);
    const float p6 = __fmul_rn(__fmul_rn(4.0f, s), wg);
    const float p7 = __fmul_rn(__fmul_rn(6.0f, s), wg);
    const uint32_t h01 = pack_f16x2_rn(p0, p1);
    const uint32_t h23 = pack_f16x2_rn(p2, p3);
    const uint32_t h45 = pack_f16x2_rn(p4, p5);
    const uint32_t h67 = pack_f16x2_rn(p6, p7);
    GroupTable t;
    t.lo0 = prmt(h01, h23, 0x6420u);
    t.lo1 = prmt(h45, h67, 0x6420u);
    t.hi0 = prmt(h01, h23, 0x7531u);
    t.hi1 = prmt(h45, h67, 0x7531u);
    return t;
}

__device__ __forceinline__ GroupTable make_group_table(uint32_t scale_byte, float wg) {
    return make_group_table_f32(e4m3_to_f32(scale_byte), wg);
}

// d = a ^ (b & c) in one logic instruction
__device__ __forceinline__ uint32_t xor_and(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x78;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Eight codes (one 32-bit word of wq: code j in bits 4j..4j+3, i.e. column order) ->
// eight f16 in column order, packed as four f16x2 words.
// The decode is bound by the integer pipe (64 lanes a clock against the FP32 pipe's 128), so the two shifts are
// written as multiplies, which the FP32 pipe's integer multiply-add takes, and each sign is folded into its
// lookup with one three-input logic instruction.
__device__ __forceinline__ void decode8(const GroupTable& t, uint32_t w, uint32_t& o0, uint32_t& o1,
                                        uint32_t& o2, uint32_t& o3) {
    const uint32_t mag = w & 0x77777777u;     // selector nibbles: bit 3 must be clear for prmt
    const uint32_t mag_hi = __umulhi(mag, 0x10000u);      // mag >> 16
    const uint32_t w4 = w * 16u;                          // w << 4
    // sign bytes: prmt's replicate-msb mode (selector bit 3) turns the sign bit of a code
    // into 0x00 / 0xff.  Codes 0..3 live in bytes 0,1 of w (odd codes: bit 7 of the byte)
    // and of w4 (even codes: bit 3 of w's byte moved up to bit 7).
    const uint32_t sgn_a = prmt(w4, w, 0xD9C8u);          // codes 0,1,2,3
    const uint32_t sgn_b = prmt(w4, w, 0xFBEAu);          // codes 4,5,6,7
    const uint32_t lo_a = prmt(t.lo0, t.lo1, mag);
    const uint32_t hi_a = xor_and(prmt(t.hi0, t.hi1, mag), sgn_a, 0x80808080u);
    const uint32_t lo_b = prmt(t.lo0, t.lo1, mag_hi);
    const uint32_t hi_b = xor_and(prmt(t.hi0, t.hi1, mag_hi), sgn_b, 0x80808080u);
    o0 = prmt(lo_a, hi_a, 0x5140u);
    o1 = prmt(lo_a, hi_a, 0x7362u);
    o2 = prmt(lo_b, hi_b, 0x5140u);
    o3 = prmt(lo_b, hi_b, 0x7362u);
}

// One group of 16 weights: q = its 8 packed bytes (q.x = columns 0-7, q.y = columns 8-15).
__device__ __forceinline__ void decode_group16(uint2 q, uint32_t scale_byte, float wg, uint4& out_lo,
                                               uint4& out_hi) {
    const GroupTable t = make_group_table(scale_byte, wg);
    decode8(t, q.x, out_lo.x, out_lo.y, out_lo.z, out_lo.w);
    decode8(t, q.y, out_hi.x, out_hi.y, out_hi.z, out_hi.w);
}

}  // namespace lexb
