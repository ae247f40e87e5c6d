// Batch 1..8 GEMV  y[b, m] = W[m, k] . x[b, k]  for bf16 or NVFP4 weights
// (config-1 operator; reference tools/analysis/nvfp4/primitive.cu:79-96 and
// experimental/weight_only_fp4/primitive.cu:22-70).
//
// Work unit = 16 output rows x one 2048-column chunk of K, one CTA of 8 warps
// per unit, warp w owning columns [w*256, +256) of the chunk.  Weights go from
// global memory straight into tensor-core A fragments (mma.sync m16n8k16, fp32
// accumulate); the up-to-8 activation vectors are the 8 columns of the B
// operand, so batch 2..8 costs no extra weight traffic or instructions.
//
//   bf16 weights : lane (g,t) loads 16 bytes of rows g and g+8 per column
//                  group; bf16 MMA against bf16 activations.
//   NVFP4 weights: lane (g,t) loads 32 code bytes and 4 scale bytes per row;
//                  codes -> f16x2 (hardware cvt), times the block scale in f16
//                  (exact: <= 6 significant bits), f16 MMA against activations
//                  converted to f16; the fp32 tensor scale is applied to the sum.
//
// K > 2048 is split across CTAs: each writes fp32 partial sums to scratch and the
// last CTA of a row block (atomic ticket) adds them in chunk order, so results
// do not depend on scheduling.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200_megakernel.h"
#include "mk_device.cuh"
#include "fp4_mma.cuh"

namespace mk {

constexpr int kGemvRows = 16;
constexpr int kGemvChunk = 2048;
constexpr int kGemvWarps = 8;
constexpr int kGemvMaxBatch = 8;

template <bool PACKED>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_mma_kernel(
    const bf16 *__restrict__ w, const uint8_t *__restrict__ packed, const uint8_t *__restrict__ scales,
    const bf16 *__restrict__ x, bf16 *__restrict__ y, int m, int k, float ts, int batch, int chunks,
    float *__restrict__ partial, int *__restrict__ tickets) {
    __shared__ float red[kGemvWarps][kGemvRows][kGemvMaxBatch];
    __shared__ int is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row_block = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const int col0 = chunk * kGemvChunk + warp * 256;  // this warp's first column
    const bool active = col0 < k;                      // k is a multiple of 256
    int row_g = row_block * kGemvRows + g, row_h = row_g + 8;
    if (row_g >= m) row_g = m - 1;                     // ragged last block: compute on a valid row, never store it
    if (row_h >= m) row_h = m - 1;
    const int xcol = g < batch ? g : batch - 1;        // B-operand column g; extra columns repeat the last vector

    // Programmatic dependent launch: the next kernel in the stream may start as soon as
    // every CTA of this one has got here, and this kernel reads its weights (which no
    // earlier kernel produces) before it waits for its predecessor.  Activations,
    // outputs and the split-K scratch are touched only after the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (!active) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (active) {
        if constexpr (PACKED) {
            uint4 cg[2], ch[2];
            const uint4 *pg = reinterpret_cast<const uint4 *>(packed + ((size_t)row_g * k + col0) / 2 + t * 32);
            const uint4 *ph = reinterpret_cast<const uint4 *>(packed + ((size_t)row_h * k + col0) / 2 + t * 32);
            cg[0] = __ldg(pg); cg[1] = __ldg(pg + 1);
            ch[0] = __ldg(ph); ch[1] = __ldg(ph + 1);
            const uint32_t sg = __ldg(reinterpret_cast<const uint32_t *>(scales + ((size_t)row_g * k + col0) / 16 + t * 4));
            const uint32_t sh = __ldg(reinterpret_cast<const uint32_t *>(scales + ((size_t)row_h * k + col0) / 16 + t * 4));
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t xh[32];
            const uint4 *xs = reinterpret_cast<const uint4 *>(x + (size_t)xcol * k + col0 + t * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 v = __ldg(xs + i);
                xh[4 * i] = bf16x2_to_f16x2(v.x); xh[4 * i + 1] = bf16x2_to_f16x2(v.y);
                xh[4 * i + 2] = bf16x2_to_f16x2(v.z); xh[4 * i + 3] = bf16x2_to_f16x2(v.w);
            }
            fp4_rows_mma(acc, cg, ch, sg, sh, xh);
        } else {
            const bf16 *wg = w + (size_t)row_g * k + col0 + t * 8;
            const bf16 *wh = w + (size_t)row_h * k + col0 + t * 8;
            const bf16 *xs = x + (size_t)xcol * k + col0 + t * 8;
            uint4 a[8], b[8], xv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                a[j] = __ldg(reinterpret_cast<const uint4 *>(wg + j * 32));
                b[j] = __ldg(reinterpret_cast<const uint4 *>(wh + j * 32));
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j) xv[j] = __ldg(reinterpret_cast<const uint4 *>(xs + j * 32));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mma_bf16_16816(acc, a[j].x, b[j].x, a[j].y, b[j].y, xv[j].x, xv[j].y);
                mma_bf16_16816(acc, a[j].z, b[j].z, a[j].w, b[j].w, xv[j].z, xv[j].w);
            }
        }
    }
    // C fragment: rows g / g+8, activation columns 2t and 2t+1
    red[warp][g][2 * t] = acc[0];
    red[warp][g][2 * t + 1] = acc[1];
    red[warp][g + 8][2 * t] = acc[2];
    red[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();

    const int r = threadIdx.x >> 3, c = threadIdx.x & 7;  // 128 threads: one (row, column) each
    float sum = 0.f;
    const bool owner = threadIdx.x < kGemvRows * kGemvMaxBatch;
    if (owner) {
#pragma unroll
        for (int wv = 0; wv < kGemvWarps; ++wv) sum += red[wv][r][c];
    }
    const int row = row_block * kGemvRows + r;
    if (chunks == 1) {
        if (owner && c < batch && row < m) y[(size_t)c * m + row] = __float2bfloat16_rn(sum * ts);
        return;
    }
    // split K: park the chunk's sums, the last chunk to arrive adds them in chunk order
    if (owner && c < batch && row < m) partial[((size_t)chunk * kGemvMaxBatch + c) * m + row] = sum;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&tickets[row_block], 1);
        is_last = ticket == chunks - 1;
        if (is_last) tickets[row_block] = 0;  // ready for the next call
        __threadfence();
    }
    __syncthreads();
    if (is_last && owner && c < batch && row < m) {
        float total = 0.f;
        for (int ch = 0; ch < chunks; ++ch) total += __ldcg(&partial[((size_t)ch * kGemvMaxBatch + c) * m + row]);
        y[(size_t)c * m + row] = __float2bfloat16_rn(total * ts);
    }
}

// Split-K scratch of mk_gemv lives in a caller-owned workspace: row-block
// tickets (ints, padded to 256 bytes) followed by the fp32 partial sums.
static size_t gemv_ticket_bytes(int m) {
    const size_t row_blocks = (size_t)(m + kGemvRows - 1) / kGemvRows;
    return (row_blocks * sizeof(int) + 255) & ~size_t(255);
}

size_t gemv_workspace_bytes(int m, int k) {
    const int chunks = (k + kGemvChunk - 1) / kGemvChunk;
    if (chunks <= 1) return 0;
    return gemv_ticket_bytes(m) + (size_t)chunks * kGemvMaxBatch * (size_t)m * sizeof(float);
}

// Launch with the programmatic-stream-serialization attribute, so that back-to-back
// GEMVs on one stream overlap one kernel's tail and the next one's start.
template <bool PACKED>
static cudaError_t launch_overlapped(dim3 grid, dim3 block, cudaStream_t stream, const bf16 *w, const uint8_t *packed,
                                     const uint8_t *scales, const bf16 *x, bf16 *y, int m, int k, float ts, int batch, int chunks,
                                     float *partial, int *tickets) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_mma_kernel<PACKED>, w, packed, scales, x, y, m, k, ts, batch, chunks, partial, tickets);
}

cudaError_t launch_gemv_mma(const void *w, const void *packed, const void *scales, const void *x, void *y, int m, int k,
                            float ts, int is_packed, int batch, void *workspace, cudaStream_t stream) {
    const int row_blocks = (m + kGemvRows - 1) / kGemvRows;
    const int chunks = (k + kGemvChunk - 1) / kGemvChunk;
    float *partial = nullptr;
    int *tickets = nullptr;
    if (chunks > 1) {
        // The tickets count arrivals per row block.  They must be zero when a call starts: the
        // caller zeroes the workspace once, and the last CTA of every row block puts its ticket
        // back to zero, so the workspace stays ready for the next call.  The partial sums are
        // written before they are read.
        tickets = reinterpret_cast<int *>(workspace);
        partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(workspace) + gemv_ticket_bytes(m));
    }
    const dim3 grid(row_blocks * chunks), block(kGemvWarps * 32);
    if (is_packed)
        return launch_overlapped<true>(grid, block, stream, nullptr, (const uint8_t *)packed, (const uint8_t *)scales, (const bf16 *)x,
                                       (bf16 *)y, m, k, ts, batch, chunks, partial, tickets);
    return launch_overlapped<false>(grid, block, stream, (const bf16 *)w, nullptr, nullptr, (const bf16 *)x, (bf16 *)y, m, k, 1.0f,
                                    batch, chunks, partial, tickets);
}

// ---------------------------------------------------------------------------
// mk_gemv_static: the same GEMV with its split-K scratch in a fixed array of the
// module instead of lazily allocated memory, so the call allocates nothing.
//
// The array holds the row-block tickets (kStaticTickets ints) followed by the
// fp32 partial sums (kStaticPartialFloats floats): 16 KiB + 4 MiB per device.
// A call needs ceil(m/16) tickets and ceil(k/2048) * 8 * m partial floats when
// k > 2048, nothing otherwise; larger problems are refused.
//
// The array is shared by every call on a device: two calls that overlap in time
// (different streams, or different threads on one stream's worth of work) race
// on it.  The first call on a device looks the array's address up, which is not
// allowed while a stream is being captured, so make it before any capture.
// ---------------------------------------------------------------------------
constexpr int kStaticTickets = 4096;
constexpr size_t kStaticPartialFloats = 1u << 20;
constexpr size_t kStaticScratchBytes = kStaticTickets * sizeof(int) + kStaticPartialFloats * sizeof(float);
static __device__ __align__(256) unsigned char g_gemv_static_scratch[kStaticScratchBytes];

static unsigned char *g_static_base[64];  // per device, filled on the first call there

void set_last_error(const char *msg);  // megakernel.cu: text for mk_last_error

static cudaError_t static_scratch(int **tickets_out, float **partial_out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (!g_static_base[device]) {
        unsigned char *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_gemv_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_base[device] = ptr;
    }
    *tickets_out = reinterpret_cast<int *>(g_static_base[device]);
    *partial_out = reinterpret_cast<float *>(g_static_base[device] + kStaticTickets * sizeof(int));
    return cudaSuccess;
}

}  // namespace mk

extern "C" int mk_gemv_static(const void *w_bf16, const void *packed, const void *scales, const void *x, void *y,
                              int32_t m, int32_t k, float tensor_scale, int32_t is_packed, int32_t batch, void *stream) {
    using namespace mk;
    if (!x || !y || m <= 0 || k <= 0 || (k % 256) != 0 || batch < 1 || batch > kGemvMaxBatch ||
        (is_packed ? (!packed || !scales) : !w_bf16)) {
        set_last_error("mk_gemv_static: null pointer, batch outside 1..8, or k not a multiple of 256");
        return MK_ERR_BAD_ARGUMENT;
    }
    const int row_blocks = (m + kGemvRows - 1) / kGemvRows;
    const int chunks = (k + kGemvChunk - 1) / kGemvChunk;
    int *tickets = nullptr;
    float *partial = nullptr;
    if (chunks > 1) {
        if (row_blocks > kStaticTickets || (size_t)chunks * kGemvMaxBatch * (size_t)m > kStaticPartialFloats) {
            char msg[256];
            snprintf(msg, sizeof(msg),
                     "mk_gemv_static: m=%d k=%d needs %d tickets and %zu partial floats; the fixed scratch holds %d and %zu "
                     "(use mk_gemv for larger problems)",
                     m, k, row_blocks, (size_t)chunks * kGemvMaxBatch * (size_t)m, kStaticTickets, kStaticPartialFloats);
            set_last_error(msg);
            return MK_ERR_UNSUPPORTED;
        }
        cudaError_t e = static_scratch(&tickets, &partial);
        if (e != cudaSuccess) {
            set_last_error("mk_gemv_static: cudaGetSymbolAddress of the fixed scratch failed (first call made during stream capture?)");
            return (int)e;
        }
        // the tickets count arrivals per row block and must start at zero; the partial sums are written before they are read
        e = cudaMemsetAsync(tickets, 0, row_blocks * sizeof(int), (cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
    }
    const dim3 grid(row_blocks * chunks), block(kGemvWarps * 32);
    if (is_packed)
        gemv_mma_kernel<true><<<grid, block, 0, (cudaStream_t)stream>>>(nullptr, (const uint8_t *)packed, (const uint8_t *)scales,
                                                                        (const bf16 *)x, (bf16 *)y, m, k, tensor_scale, batch,
                                                                        chunks, partial, tickets);
    else
        gemv_mma_kernel<false><<<grid, block, 0, (cudaStream_t)stream>>>((const bf16 *)w_bf16, nullptr, nullptr, (const bf16 *)x,
                                                                         (bf16 *)y, m, k, 1.0f, batch, chunks, partial, tickets);
    return (int)cudaGetLastError();
}
