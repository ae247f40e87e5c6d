// Batched decode linear  y[b, n] = sum_k x[b, k] * W[n, k]  for 16..128 sequences
// on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// This is the dense-contraction counterpart of the batch-1 megakernel's matvec
// tiles: once a decode step carries 16 or more sequences, one weight row meets a
// [K, batch] activation panel and the op is a GEMM with a small N.  The
// reference's operator for this is include/ops/nvfp4_linear.cuh:52-173 (TMA
// operand staging, tcgen05.mma, tcgen05.ld epilogue).
//
// Shape of the work.  Weights are the A operand: a CTA owns a slab of 128 weight
// rows (the MMA's M, one row per tensor-memory lane) and a range of K blocks;
// the activations are the B operand with N = batch padded to 16/32/64/128.  The
// accumulator D[128 rows, batch] lives in tensor memory, double buffered so that
// the epilogue of one slab overlaps the MMAs of the next.  Per K block of 64
// columns, TMA (cp.async.bulk.tensor, 128-byte swizzle) brings a 128 x 64 weight
// tile (16 KiB) and the batch x 64 activation tile into a shared-memory ring; one
// elected thread issues four K=16 MMAs per block and commits the stage back to
// the loader.  Weights are read from HBM exactly once; the activation panel
// (at most 2 MiB) is re-read from L2.
//
// Warp roles (192 threads): warp 0 loader (one lane), warp 1 tensor-memory
// allocation + MMA issue (one lane), warps 2-5 epilogue (tensor-memory lane
// quarter = warp index mod 4): tcgen05.ld, bf16 conversion, transposed store
// y[b, row].  With split-K (narrow matrices that would otherwise occupy few SMs)
// the epilogue writes fp32 partial sums [split, batch, n] for the caller's next
// kernel to add in split order.
//
// Every wait is bounded: on expiry the CTA sets an error word, skips the rest of
// its work, waits (bounded) for copies in flight, frees its tensor memory and
// returns.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200_megakernel.h"
#include "mk_device.cuh"

namespace mk {

void set_last_error(const char *msg);  // megakernel.cu: text for mk_last_error

namespace lb {

constexpr int kSlabRows = 128;          // MMA M: weight rows per slab
constexpr int kBlockK = 64;             // bf16 columns per stage: one 128-byte swizzle row
constexpr int kUmmaK = 16;              // K of one tcgen05.mma for 16-bit operands
constexpr int kThreads = 192;
constexpr int kATileBytes = kSlabRows * kBlockK * 2;  // 16 KiB
constexpr int kMaxBatch = 128;
constexpr long long kWaitCycles = 2000000000ll;       // about a second

struct __align__(1024) Stage {
    uint8_t a[kATileBytes];
    uint8_t b[kMaxBatch * kBlockK * 2];
};

template <int STAGES>
struct Smem {
    Stage stage[STAGES];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int failed;
};

struct Params {
    int n, k, batch, batch_pad;   // batch_pad: MMA N, power of two in 16..128
    int splits, kblocks_per_split;
    int slabs;
    bf16 *y;                      // [batch, n] when splits == 1
    float *partials;              // [splits, batch, n] otherwise
    int *error;                   // device word: non-zero when a wait ran out
};

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity, volatile int *failed) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned it = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++it & 63u) == 0) {
            if (*failed) return false;
            if (clock64() - t0 > kWaitCycles) {
                *failed = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (one swizzle row): start address, 8-row groups 1024 bytes apart, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(const void *tile) {
    const uint64_t addr = smem_addr(tile);
    return ((addr >> 4) & 0x3fffull) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kSlabRows >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on the barrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 16 consecutive fp32 columns of tensor memory: thread i gets lane (base lane + i).
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
linear_batched_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem<STAGES> &s = *reinterpret_cast<Smem<STAGES> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *failed = &s.failed;
    const uint32_t acc_cols = (uint32_t)p.batch_pad;       // fp32 columns of one accumulator
    const uint32_t tmem_cols = acc_cols * 2 < 32 ? 32 : acc_cols * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], 4);  // one arrival per epilogue warp
        }
        s.failed = 0;
        fence_barrier_init();
    }
    if (warp == 1) {  // one whole warp allocates tensor memory and later frees it
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s.tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = s.tmem_base;

    // work items of this CTA: (slab, split) pairs, dealt round robin
    const int items = p.slabs * p.splits;
    const int stage_tx = kATileBytes + p.batch_pad * kBlockK * 2;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t stream_policy = l2_evict_first_policy();  // weights: read once
            uint64_t keep_policy;                                    // activations: re-read by every CTA
            asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_policy));
            uint32_t stage = 0, phase = 0, filled = 0;  // filled: stages that have been filled at least once
            for (int item = blockIdx.x; item < items && !*failed; item += gridDim.x) {
                const int slab = item / p.splits, split = item % p.splits;
                const int kb0 = split * p.kblocks_per_split;
                for (int kb = kb0; kb < kb0 + p.kblocks_per_split; ++kb) {
                    if (!wait_bounded(&s.empty[stage], phase ^ 1u, failed)) break;
                    filled |= 1u << stage;
                    mbar_arrive_expect_tx(&s.full[stage], stage_tx);
                    tma_load_2d(s.stage[stage].a, &map_w, kb * kBlockK, slab * kSlabRows, &s.full[stage], stream_policy);
                    tma_load_2d(s.stage[stage].b, &map_x, kb * kBlockK, 0, &s.full[stage], keep_policy);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            // Never leave with copies in flight.  In a clean run the MMA warp has waited for every
            // fill; after a failure, wait here (bounded) for the most recent fill of every stage.
            if (*failed) {
                for (uint32_t i = 0; i < (uint32_t)STAGES; ++i) {
                    if (!(filled & (1u << i))) continue;
                    const uint32_t parity = i < stage ? phase : (phase ^ 1u);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(&s.full[i], parity)) {
                        if (clock64() - t0 > kWaitCycles) break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16(p.batch_pad);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            for (int item = blockIdx.x; item < items && !*failed; item += gridDim.x) {
                if (!wait_bounded(&s.acc_empty[acc], acc_phase ^ 1u, failed)) break;
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * acc_cols;
                bool ok = true;
                for (int kb = 0; kb < p.kblocks_per_split && ok; ++kb) {
                    ok = wait_bounded(&s.full[stage], phase, failed);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint64_t da = smem_desc_k_major_sw128(s.stage[stage].a);
                    const uint64_t db = smem_desc_k_major_sw128(s.stage[stage].b);
#pragma unroll
                    for (int ks = 0; ks < kBlockK / kUmmaK; ++ks)  // 32 bytes further along the swizzled row per K step
                        umma_bf16(tmem_d, da + 2 * ks, db + 2 * ks, idesc, (kb | ks) != 0);
                    umma_commit(&s.empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&s.acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // epilogue: warp w may touch tensor-memory lanes 32*(w % 4) .. +31
        const int quarter = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int slab = item / p.splits, split = item % p.splits;
            bool ok = wait_bounded(&s.acc_full[acc], acc_phase, failed);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const int row = slab * kSlabRows + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * acc_cols;
            for (int c0 = 0; c0 < p.batch_pad; c0 += 16) {
                uint32_t v[16];
                tmem_load16(taddr + c0, v);
                if (row < p.n) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = c0 + j;
                        if (b < p.batch) {
                            if (p.splits == 1) p.y[(size_t)b * p.n + row] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            else p.partials[((size_t)split * p.batch + b) * p.n + row] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.acc_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (threadIdx.x == 0 && s.failed) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// bf16 matrix [rows, k] row-major -> boxes of 64 columns x box_rows rows, 128-byte swizzle
static bool make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t k, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int kStages = 6;

}  // namespace lb
}  // namespace mk

extern "C" int32_t mk_linear_batched_splits(int32_t n, int32_t k, int32_t sm_count) {
    // Enough (slab, split) items to give every SM work, while a split keeps at least 8 K blocks.
    if (n <= 0 || k <= 0 || sm_count <= 0) return 1;
    const int slabs = (n + mk::lb::kSlabRows - 1) / mk::lb::kSlabRows, kblocks = k / mk::lb::kBlockK;
    int splits = 1;
    while (slabs * splits < sm_count && kblocks % (splits * 2) == 0 && kblocks / (splits * 2) >= 8) splits *= 2;
    return splits;
}

extern "C" int mk_linear_batched(const void *w_bf16, const void *x_bf16, void *y_bf16, float *partials, int32_t n, int32_t k,
                                 int32_t batch, int32_t splits, int32_t *error_word, void *stream) {
    using namespace mk;
    using namespace mk::lb;
    char msg[256];
    if (!w_bf16 || !x_bf16 || n <= 0 || k <= 0 || batch < 1 || batch > kMaxBatch || splits < 1 || !error_word ||
        (splits == 1 ? !y_bf16 : !partials)) {
        set_last_error("mk_linear_batched: null pointer, batch outside 1..128 or splits < 1");
        return MK_ERR_BAD_ARGUMENT;
    }
    if (k % kBlockK || (k / kBlockK) % splits || (reinterpret_cast<uintptr_t>(w_bf16) & 15) || (reinterpret_cast<uintptr_t>(x_bf16) & 15)) {
        snprintf(msg, sizeof(msg), "mk_linear_batched: k=%d must be a multiple of 64 and of 64*splits (%d); pointers 16-byte aligned", k, splits);
        set_last_error(msg);
        return MK_ERR_UNSUPPORTED;
    }
    int batch_pad = 16;
    while (batch_pad < batch) batch_pad *= 2;
    CUtensorMap map_w, map_x;
    // rows beyond n / batch are outside the tensor: TMA fills them with zeros
    if (!make_map(&map_w, w_bf16, (uint64_t)n, (uint64_t)k, kSlabRows) || !make_map(&map_x, x_bf16, (uint64_t)batch, (uint64_t)k, (uint32_t)batch_pad)) {
        set_last_error("mk_linear_batched: cuTensorMapEncodeTiled failed (driver without tensor-map support?)");
        return MK_ERR_UNSUPPORTED;
    }
    Params p;
    p.n = n; p.k = k; p.batch = batch; p.batch_pad = batch_pad;
    p.splits = splits; p.kblocks_per_split = (k / kBlockK) / splits;
    p.slabs = (n + kSlabRows - 1) / kSlabRows;
    p.y = (bf16 *)y_bf16; p.partials = partials; p.error = error_word;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    const size_t smem = sizeof(Smem<kStages>) + 1024;
    static bool configured[64] = {};
    if (device < 64 && !configured[device]) {
        e = cudaFuncSetAttribute(linear_batched_kernel<kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    const int items = p.slabs * splits;
    const int grid = items < sms ? items : sms;
    linear_batched_kernel<kStages><<<grid, kThreads, smem, (cudaStream_t)stream>>>(map_w, map_x, p);
    return (int)cudaGetLastError();
}
