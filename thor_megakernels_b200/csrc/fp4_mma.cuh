// Tensor-core building blocks shared by the GEMV kernel and the decode
// megakernel: warp-level MMA wrappers and the NVFP4 -> f16 operand decode.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "mk_device.cuh"

namespace mk {

// D += A(16x16) * B(16x8), fp32 accumulate.  volatile keeps hand-written
// load/MMA interleavings in program order.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two E2M1 codes (one byte) -> f16x2, low nibble first.
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Four E2M1 codes -> two f16x2 (codes 0,1 and codes 2,3), by table look-up: the
// magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 are f16 values whose low byte is zero, so
// one byte permute with the 3-bit magnitudes as selectors fetches the four high
// bytes at once; a second permute in sign-replication mode turns the codes' sign
// bits into byte masks.  `w` holds eight codes, `w4 = w << 4`, `half` picks codes
// 0..3 or 4..7 of the word.
__device__ __forceinline__ void e2m1x4_to_f16x4(uint32_t w, uint32_t w4, int half, uint32_t &p01, uint32_t &p23) {
    const uint32_t sel = (half ? (w >> 16) : w) & 0x7777u;
    const uint32_t mag = prmt(0x3E3C3800u, 0x46444240u, sel);
    // even codes have their sign in bit 7 of a byte of w4, odd codes in bit 7 of a byte of w
    const uint32_t sign = prmt(w, w4, half ? 0xBFAEu : 0x9D8Cu);
    const uint32_t hb = mag | (sign & 0x80808080u);
    p01 = prmt(hb, 0u, 0x1404u);
    p23 = prmt(hb, 0u, 0x3424u);
}

// One E4M3 scale byte -> the same f16 value in both halves.
__device__ __forceinline__ uint32_t e4m3_to_f16x2_dup(uint32_t byte) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xffu), __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.x << 16);
}

__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Two bf16 (packed) -> two f16 (packed).  Exact for 2^-14 <= |x| <= 65504;
// larger magnitudes are clamped to +-65504 (the largest finite f16) instead of
// becoming infinite, smaller ones lose bits and flush to zero below 2^-24.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    const float lo = fminf(fmaxf(bf16_lo(v), -65504.f), 65504.f), hi = fminf(fmaxf(bf16_hi(v), -65504.f), 65504.f);
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// 16 rows x 256 columns of NVFP4 weights (this warp's share of a chunk) times
// the activation columns, accumulated into acc.  codes_g/codes_h: the lane's 32
// code bytes of rows g and g+8 (columns t*64 .. t*64+63 of the warp's range);
// sc_g/sc_h: the 4 scale bytes of those columns; xh: the lane's 64 activation
// values as f16 pairs, in the same column order.
__device__ __forceinline__ void fp4_rows_mma(float (&acc)[4], const uint4 (&codes_g)[2], const uint4 (&codes_h)[2],
                                             uint32_t sc_g, uint32_t sc_h, const uint32_t (&xh)[32]) {
    const uint32_t wg[8] = {codes_g[0].x, codes_g[0].y, codes_g[0].z, codes_g[0].w,
                            codes_g[1].x, codes_g[1].y, codes_g[1].z, codes_g[1].w};
    const uint32_t wh[8] = {codes_h[0].x, codes_h[0].y, codes_h[0].z, codes_h[0].w,
                            codes_h[1].x, codes_h[1].y, codes_h[1].z, codes_h[1].w};
    float acc2[4] = {0.f, 0.f, 0.f, 0.f};  // second accumulator: halves the chain of dependent MMAs
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {  // one 16-column scale block = 8 code bytes = 2 words
        const uint32_t sg = e4m3_to_f16x2_dup(sc_g >> (8 * blk));
        const uint32_t sh = e4m3_to_f16x2_dup(sc_h >> (8 * blk));
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint32_t cg = wg[2 * blk + half], ch = wh[2 * blk + half];
            const uint32_t cg4 = cg << 4, ch4 = ch << 4;
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {  // an MMA takes 2 bytes (4 codes) per row
                const int i = (2 * blk + half) * 2 + pair;  // MMA index 0..15, columns 4i..4i+3 of the lane
                uint32_t g01, g23, h01, h23;
                e2m1x4_to_f16x4(cg, cg4, pair, g01, g23);
                e2m1x4_to_f16x4(ch, ch4, pair, h01, h23);
                const uint32_t a0 = hmul2_bits(g01, sg), a2 = hmul2_bits(g23, sg);
                const uint32_t a1 = hmul2_bits(h01, sh), a3 = hmul2_bits(h23, sh);
                if (i & 1) mma_f16_16816(acc2, a0, a1, a2, a3, xh[2 * i], xh[2 * i + 1]);
                else mma_f16_16816(acc, a0, a1, a2, a3, xh[2 * i], xh[2 * i + 1]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[r] += acc2[r];
}

// Same, with the activation operand kept as eight 16-byte vectors.
__device__ __forceinline__ void fp4_rows_mma(float (&acc)[4], const uint4 (&codes_g)[2], const uint4 (&codes_h)[2],
                                             uint32_t sc_g, uint32_t sc_h, const uint4 (&x)[8]) {
    uint32_t xh[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        xh[4 * i] = x[i].x; xh[4 * i + 1] = x[i].y; xh[4 * i + 2] = x[i].z; xh[4 * i + 3] = x[i].w;
    }
    fp4_rows_mma(acc, codes_g, codes_h, sc_g, sc_h, xh);
}

}  // namespace mk
