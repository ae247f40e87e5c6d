// NVFP4 weight format: quantiser and weight-only GEMV (sm_100a).
//
// Format (reference tools/analysis/nvfp4/primitive.cu:50-75): for a bf16 matrix
// [rows, k] and a per-tensor fp32 scale ts, every 16 consecutive k values v =
// w / ts share one E4M3 scale sf = e4m3(max(amax(v) / 6, 2^-9)); each value is
// stored as the E2M1 code of v / float(sf), two codes per byte with the even
// element in the low nibble.  Dequantised weight = e2m1(code) * float(sf) * ts.

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200_megakernel.h"
#include "mk_device.cuh"

namespace mk {

// One thread quantises one 16-value group: 32 B in, 8 B codes + 1 B scale out.
__global__ void nvfp4_quantize_kernel(const bf16 *__restrict__ input, uint8_t *__restrict__ packed,
                                      uint8_t *__restrict__ scales, float *__restrict__ decoded, long long groups,
                                      float tensor_scale) {
    const long long grp = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (grp >= groups) return;
    const uint4 *src = reinterpret_cast<const uint4 *>(input + grp * 16);
    float v[16];
    {
        float a[8], b[8];
        unpack8(__ldg(src), a);
        unpack8(__ldg(src + 1), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = a[i] / tensor_scale;
            v[8 + i] = b[i] / tensor_scale;
        }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // round the block scale first, then quantise against the rounded scale
    const __nv_fp8_e4m3 sf(fmaxf(amax / 6.f, 1.f / 512.f));
    const float scale = float(sf);
    uint32_t lo = 0, hi = 0;
    uint8_t q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = (uint8_t)__nv_cvt_float_to_fp4(v[i] / scale, __NV_E2M1, cudaRoundNearest) & 0xF;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo |= (uint32_t)(q[2 * i] | (q[2 * i + 1] << 4)) << (8 * i);
        hi |= (uint32_t)(q[8 + 2 * i] | (q[8 + 2 * i + 1] << 4)) << (8 * i);
    }
    *reinterpret_cast<uint2 *>(packed + grp * 8) = make_uint2(lo, hi);
    scales[grp] = sf.__x;
    if (decoded) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __half_raw h = __nv_cvt_fp4_to_halfraw(q[i], __NV_E2M1);
            decoded[grp * 16 + i] = __half2float(__half(h)) * scale * tensor_scale;
        }
    }
}

// e2m1 code -> value.  Codes 0..7 = 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
    return __half22float2(__half2(h));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t bits) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)bits, __NV_E4M3);
    return __half2float(__half(h));
}

// Warp per output row, lanes stride over K, fp32 accumulation, shuffle
// reduction (reference primitive.cu:79-96), for up to 8 activation vectors.
// Each lane step covers 32 columns: 16 B of codes and two scale bytes, or 64 B
// of bf16 weights.
template <bool PACKED, int BATCH>
__global__ void __launch_bounds__(256) gemv_kernel(const bf16 *__restrict__ w, const uint8_t *__restrict__ packed,
                                                   const uint8_t *__restrict__ scales, const bf16 *__restrict__ x,
                                                   bf16 *__restrict__ y, int m, int k, float ts) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < m; row += warps_total) {
        float acc[BATCH];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) acc[b] = 0.f;
        for (int c = lane * 32; c < k; c += 32 * 32) {
            float wv[32];
            if constexpr (PACKED) {
                const uint4 codes = __ldg(reinterpret_cast<const uint4 *>(packed + ((size_t)row * k + c) / 2));
                const unsigned short sc2 = __ldg(reinterpret_cast<const unsigned short *>(scales + (size_t)row * (k / 16) + c / 16));
                const float s0 = e4m3_to_float(sc2 & 0xff) * ts, s1 = e4m3_to_float(sc2 >> 8) * ts;
                const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 f = e2m1x2_to_float2((words[i >> 2] >> (8 * (i & 3))) & 0xff);
                    const float s = i < 8 ? s0 : s1;
                    wv[2 * i] = f.x * s;
                    wv[2 * i + 1] = f.y * s;
                }
            } else {
                const uint4 *src = reinterpret_cast<const uint4 *>(w + (size_t)row * k + c);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float t[8];
                    unpack8(__ldg(src + i), t);
#pragma unroll
                    for (int j = 0; j < 8; ++j) wv[8 * i + j] = t[j];
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const uint4 *xs = reinterpret_cast<const uint4 *>(x + (size_t)b * k + c);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float t[8];
                    unpack8(__ldg(xs + i), t);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[b] = fmaf(wv[8 * i + j], t[j], acc[b]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            float v = acc[b];
#pragma unroll
            for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0) y[(size_t)b * m + row] = __float2bfloat16_rn(v);
        }
    }
}

template <bool PACKED>
static cudaError_t launch_gemv(const void *w, const void *packed, const void *scales, const void *x, void *y, int m,
                               int k, float ts, int batch, cudaStream_t stream) {
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int warps_per_cta = 8;
    int ctas = (m + warps_per_cta - 1) / warps_per_cta;
    const int cap = sms * 8;
    if (ctas > cap) ctas = cap;
#define MK_GEMV_CASE(B)                                                                                              \
    case B:                                                                                                          \
        gemv_kernel<PACKED, B><<<ctas, 256, 0, stream>>>((const bf16 *)w, (const uint8_t *)packed,                   \
                                                         (const uint8_t *)scales, (const bf16 *)x, (bf16 *)y, m, k, ts); \
        break;
    switch (batch) {
        MK_GEMV_CASE(1) MK_GEMV_CASE(2) MK_GEMV_CASE(3) MK_GEMV_CASE(4)
        MK_GEMV_CASE(5) MK_GEMV_CASE(6) MK_GEMV_CASE(7) MK_GEMV_CASE(8)
    default:
        return cudaErrorInvalidValue;
    }
#undef MK_GEMV_CASE
    return cudaGetLastError();
}

// tensor-core path (gemv.cu); needs k to be a multiple of 256
cudaError_t launch_gemv_mma(const void *w, const void *packed, const void *scales, const void *x, void *y, int m, int k,
                            float ts, int is_packed, int batch, void *workspace, cudaStream_t stream);
size_t gemv_workspace_bytes(int m, int k);
void set_last_error(const char *msg);  // megakernel.cu: text for mk_last_error

}  // namespace mk

extern "C" int mk_nvfp4_quantize(const void *input_bf16, void *packed, void *scales, float *decoded, int32_t rows,
                                 int32_t k, float tensor_scale, void *stream) {
    if (!input_bf16 || !packed || !scales || rows <= 0 || k <= 0 || (k % 16) != 0 || !(tensor_scale > 0.f))
        return cudaErrorInvalidValue;
    const long long groups = (long long)rows * (k / 16);
    const int threads = 256;
    const long long blocks = (groups + threads - 1) / threads;
    mk::nvfp4_quantize_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        (const mk::bf16 *)input_bf16, (uint8_t *)packed, (uint8_t *)scales, decoded, groups, tensor_scale);
    return (int)cudaGetLastError();
}

extern "C" int64_t mk_gemv_workspace_bytes(int32_t m, int32_t k) {
    if (m <= 0 || k <= 0 || (k % 256) != 0) return 0;  // widths that are not a multiple of 256 run without scratch
    return (int64_t)mk::gemv_workspace_bytes(m, k);
}

extern "C" int mk_gemv(const void *w_bf16, const void *packed, const void *scales, const void *x, void *y, int32_t m,
                       int32_t k, float tensor_scale, int32_t is_packed, int32_t batch, void *workspace,
                       int64_t workspace_bytes, void *stream) {
    if (!x || !y || m <= 0 || k <= 0 || (k % 32) != 0 || batch < 1 || batch > 8) return cudaErrorInvalidValue;
    if (is_packed ? (!packed || !scales) : !w_bf16) return cudaErrorInvalidValue;
    if (k % 256 == 0) {
        const int64_t need = (int64_t)mk::gemv_workspace_bytes(m, k);
        if (need > 0 && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))) {
            char msg[200];
            snprintf(msg, sizeof(msg), "mk_gemv: m=%d k=%d needs a 256-byte aligned workspace of %lld bytes (mk_gemv_workspace_bytes), got %lld",
                     m, k, (long long)need, (long long)(workspace ? workspace_bytes : 0));
            mk::set_last_error(msg);
            return MK_ERR_BAD_ARGUMENT;
        }
        return (int)mk::launch_gemv_mma(w_bf16, packed, scales, x, y, m, k, tensor_scale, is_packed, batch, workspace,
                                        (cudaStream_t)stream);
    }
    // odd widths: plain warp-per-row kernel
    if (is_packed) {
        return (int)mk::launch_gemv<true>(nullptr, packed, scales, x, y, m, k, tensor_scale, batch, (cudaStream_t)stream);
    }
    if (!w_bf16) return cudaErrorInvalidValue;
    return (int)mk::launch_gemv<false>(w_bf16, nullptr, nullptr, x, y, m, k, 1.0f, batch, (cudaStream_t)stream);
}
