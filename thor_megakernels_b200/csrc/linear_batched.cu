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
// NVFP4 variant (kind::mxf4nvf4, block16): both operands are E2M1 codes, two per
// byte, with one UE4M3 scale per 16 consecutive K (reference
// include/ops/nvfp4_linear.cuh:52-173).  A stage then covers 256 columns of K
// (still one 128-byte swizzle row), and carries the 128 x 16 block scales of the
// weight slab and of the activation panel (2 KiB each, stored in global memory
// in the 512-byte atoms the tensor core reads: 32 rows x 16 bytes, byte
// (r % 32) * 16 + (r % 128 / 32) * 4 + g % 4 for row r and K group g).  Before a
// stage's four K=64 MMAs the issuing thread copies the scales from shared to
// tensor memory (tcgen05.cp 32x128b.warpx4); the MMA applies them.  The epilogue
// multiplies by the two fp32 tensor scales.
//
// Every wait is bounded: on expiry the CTA sets an error word, skips the rest of
// its work, waits (bounded) for copies in flight, frees its tensor memory and
// returns.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200_megakernel.h"
#include "mk_device.cuh"
#include "batched_ops.cuh"
#include "tma_host.cuh"

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

constexpr int kSfBytes = 2048;          // block scales of 128 rows x 256 columns (4 atoms of 512 bytes)

template <bool FP4>
struct __align__(1024) Stage {
    uint8_t a[kATileBytes];
    uint8_t b[kMaxBatch * kBlockK * 2];
    uint8_t sfa[FP4 ? kSfBytes : 16];
    uint8_t sfb[FP4 ? kSfBytes : 16];
};

template <int STAGES, bool FP4>
struct Smem {
    Stage<FP4> stage[STAGES];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int failed;
};

struct Params {
    int n, k, batch, batch_pad;   // batch_pad: MMA N, power of two in 16..128
    int splits, kblocks_per_split;  // K blocks: 64 columns (bf16) or 256 columns (NVFP4)
    int kblocks;                  // K blocks of the whole matrix
    const uint8_t *sfa, *sfb;     // NVFP4: block scales of weights / activations in 512-byte atoms
    float alpha;                  // NVFP4: weight tensor scale x activation tensor scale
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

// kind::mxf4nvf4 instruction descriptor: E2M1 x E2M1, UE4M3 scales per 16, fp32 accumulate, M = 128, K = 64.
__device__ __forceinline__ uint32_t idesc_nvfp4(int n) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kSlabRows >> 4) << 24);
}

__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                           uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// One 512-byte scale atom (32 rows x 16 bytes, dense) from shared to tensor memory:
// lane L of every 32-lane quarter receives row L % 32, i.e. 4 columns of 32 bits.
__device__ __forceinline__ void copy_scales_to_tmem(uint32_t taddr, const void *atom) {
    const uint64_t addr = smem_addr(atom);
    // no swizzle, 8-row groups 128 bytes apart, one 16-byte column
    const uint64_t desc = ((addr >> 4) & 0x3fffull) | (8ull << 32) | (1ull << 46);
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
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

template <int STAGES, bool FP4>
__global__ void __launch_bounds__(kThreads, 1)
linear_batched_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem<STAGES, FP4> &s = *reinterpret_cast<Smem<STAGES, FP4> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // K columns per stage and their bytes in a 128-byte swizzle row: 64 bf16 or 256 four-bit codes
    constexpr int kStageK = FP4 ? 256 : kBlockK;
    static_assert(kStageK == 64 || kStageK == 256, "one 128-byte swizzle row per stage");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *failed = &s.failed;
    pdl_launch_dependents();  // the next kernel on the stream may start its own prologue
    const uint32_t acc_cols = (uint32_t)p.batch_pad;       // fp32 columns of one accumulator
    // two accumulators, then (NVFP4) 16 columns of weight scales and 16 of activation scales
    const uint32_t sf_base = acc_cols * 2;
    uint32_t tmem_cols = 32;
    while (tmem_cols < acc_cols * 2 + (FP4 ? 32u : 0u)) tmem_cols *= 2;

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
    const int stage_tx = kATileBytes + p.batch_pad * kBlockK * 2 + (FP4 ? 2 * kSfBytes : 0);

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t stream_policy = l2_evict_first_policy();  // weights: read once
            uint64_t keep_policy;                                    // activations: re-read by every CTA
            asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_policy));
            uint32_t stage = 0, phase = 0, filled = 0;  // filled: stages that have been filled at least once
            // fills in order: (item, K block) pairs of this CTA
            struct Fill { int item, kb, kb_end; };
            auto first_fill = [&]() {
                Fill f{(int)blockIdx.x, 0, 0};
                if (f.item < items) { f.kb = (f.item % p.splits) * p.kblocks_per_split; f.kb_end = f.kb + p.kblocks_per_split; }
                return f;
            };
            auto next_fill = [&](Fill &f) {
                if (++f.kb == f.kb_end) {
                    f.item += gridDim.x;
                    if (f.item < items) { f.kb = (f.item % p.splits) * p.kblocks_per_split; f.kb_end = f.kb + p.kblocks_per_split; }
                }
            };
            // weights (and their scales) do not depend on the kernel before this one; activations do
            auto load_weights = [&](const Fill &f, uint32_t st) {
                const int slab = f.item / p.splits;
                const int x = FP4 ? f.kb * 128 : f.kb * kBlockK;  // bf16 columns, or bytes of packed codes (128 per stage)
                tma_load_2d(s.stage[st].a, &map_w, x, slab * kSlabRows, &s.full[st], stream_policy);
                if constexpr (FP4)
                    bulk_load(s.stage[st].sfa, p.sfa + ((size_t)slab * p.kblocks + f.kb) * kSfBytes, kSfBytes, &s.full[st], stream_policy);
            };
            auto load_activations = [&](const Fill &f, uint32_t st) {
                const int x = FP4 ? f.kb * 128 : f.kb * kBlockK;
                tma_load_2d(s.stage[st].b, &map_x, x, 0, &s.full[st], keep_policy);
                if constexpr (FP4) bulk_load(s.stage[st].sfb, p.sfb + (size_t)f.kb * kSfBytes, kSfBytes, &s.full[st], keep_policy);
            };
            // Prologue: the weight tiles of the first STAGES fills are requested before the
            // predecessor kernel has finished (every stage is free at the start); their
            // activation tiles follow once it has.
            Fill f = first_fill();
            {
                Fill g = f;
                int n = 0;
                for (; n < STAGES && g.item < items; ++n, next_fill(g)) {
                    filled |= 1u << n;
                    mbar_arrive_expect_tx(&s.full[n], stage_tx);
                    load_weights(g, n);
                }
                pdl_wait();
                for (int i = 0; i < n; ++i, next_fill(f)) load_activations(f, i);
                stage = n == STAGES ? 0 : n;
                phase = n == STAGES ? 1u : 0u;
            }
            for (; f.item < items && !*failed; next_fill(f)) {
                if (!wait_bounded(&s.empty[stage], phase ^ 1u, failed)) break;
                filled |= 1u << stage;
                mbar_arrive_expect_tx(&s.full[stage], stage_tx);
                load_weights(f, stage);
                load_activations(f, stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
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
            const uint32_t idesc = FP4 ? idesc_nvfp4(p.batch_pad) : idesc_bf16(p.batch_pad);
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
                    if constexpr (FP4) {
                        // this stage's scales: 4 atoms each for the weight slab and the activation panel
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            copy_scales_to_tmem(tmem_base + sf_base + 4 * ks, s.stage[stage].sfa + 512 * ks);
                            copy_scales_to_tmem(tmem_base + sf_base + 16 + 4 * ks, s.stage[stage].sfb + 512 * ks);
                        }
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)  // K = 64 codes = 32 bytes further along the swizzled row per step
                            umma_nvfp4(tmem_d, da + 2 * ks, db + 2 * ks, idesc, (kb | ks) != 0, tmem_base + sf_base + 4 * ks,
                                       tmem_base + sf_base + 16 + 4 * ks);
                    } else {
#pragma unroll
                        for (int ks = 0; ks < kBlockK / kUmmaK; ++ks)  // 32 bytes further along the swizzled row per K step
                            umma_bf16(tmem_d, da + 2 * ks, db + 2 * ks, idesc, (kb | ks) != 0);
                    }
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
        pdl_wait();  // the output buffer may still be read by the kernels before this one
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
                            const float value = FP4 ? __uint_as_float(v[j]) * p.alpha : __uint_as_float(v[j]);
                            if (p.splits == 1) p.y[(size_t)b * p.n + row] = __float2bfloat16_rn(value);
                            else p.partials[((size_t)split * p.batch + b) * p.n + row] = value;
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

// Row-major matrix [rows, row_bytes] -> boxes of 128 bytes x box_rows rows, 128-byte swizzle.
// bf16: 64 elements per box row; packed E2M1 codes are moved as bytes (256 codes per box row).
static bool make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, bool bytes) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {bytes ? row_bytes : row_bytes / 2, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {bytes ? 128u : 64u, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int kStagesBf16 = 6;   // 6 x 32 KiB
constexpr int kStagesFp4 = 5;    // 5 x 36 KiB

template <bool FP4>
static int launch(const void *w, const void *x, const uint8_t *sfa, const uint8_t *sfb, float alpha, void *y, float *partials,
                  int n, int k, int batch, int splits, int *error_word, cudaStream_t stream, const char *who) {
    constexpr int kStages = FP4 ? kStagesFp4 : kStagesBf16;
    constexpr int kStageK = FP4 ? 256 : kBlockK;
    char msg[256];
    if (!w || !x || n <= 0 || k <= 0 || batch < 1 || batch > kMaxBatch || splits < 1 || !error_word || (splits == 1 ? !y : !partials) ||
        (FP4 && (!sfa || !sfb))) {
        snprintf(msg, sizeof(msg), "%s: null pointer, batch outside 1..128 or splits < 1", who);
        set_last_error(msg);
        return MK_ERR_BAD_ARGUMENT;
    }
    if (k % kStageK || (k / kStageK) % splits || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (FP4 && ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)))) {
        snprintf(msg, sizeof(msg), "%s: k=%d must be a multiple of %d and of %d*splits (%d); pointers 16-byte aligned", who, k, kStageK,
                 kStageK, splits);
        set_last_error(msg);
        return MK_ERR_UNSUPPORTED;
    }
    int batch_pad = 16;
    while (batch_pad < batch) batch_pad *= 2;
    const uint64_t row_bytes = FP4 ? (uint64_t)k / 2 : (uint64_t)k * 2;
    CUtensorMap map_w, map_x;
    // rows beyond n / batch are outside the tensor: TMA fills them with zeros
    if (!make_map(&map_w, w, (uint64_t)n, row_bytes, kSlabRows, FP4) || !make_map(&map_x, x, (uint64_t)batch, row_bytes, (uint32_t)batch_pad, FP4)) {
        snprintf(msg, sizeof(msg), "%s: cuTensorMapEncodeTiled failed (driver without tensor-map support?)", who);
        set_last_error(msg);
        return MK_ERR_UNSUPPORTED;
    }
    Params p;
    p.n = n; p.k = k; p.batch = batch; p.batch_pad = batch_pad;
    p.kblocks = k / kStageK;
    p.splits = splits; p.kblocks_per_split = p.kblocks / splits;
    p.slabs = (n + kSlabRows - 1) / kSlabRows;
    p.y = (bf16 *)y; p.partials = partials; p.error = error_word;
    p.sfa = sfa; p.sfb = sfb; p.alpha = alpha;
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    const size_t smem = sizeof(Smem<kStages, FP4>) + 1024;
    static bool configured[64] = {};
    if (device < 64 && !configured[device]) {
        e = cudaFuncSetAttribute(linear_batched_kernel<kStages, FP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    const int items = p.slabs * splits;
    const int grid = items < sms ? items : sms;
    e = launch_pdl(linear_batched_kernel<kStages, FP4>, dim3(grid), dim3(kThreads), smem, stream, map_w, map_x, p);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

// One thread quantises 16 consecutive values of a row (the arithmetic of the
// weight quantiser, nvfp4.cu: v = x / tensor_scale, scale = e4m3(max(amax / 6, 2^-9)),
// code = e2m1(v / scale)); codes go to packed [rows, k/2], the scale byte into the
// 512-byte atoms the tensor core reads.
__global__ void quantize_native_kernel(const bf16 *__restrict__ input, uint8_t *__restrict__ packed, uint8_t *__restrict__ sf,
                                       int rows, int k, float tensor_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups_per_row = k / 16;
    const long long grp = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (grp >= (long long)rows * groups_per_row) return;
    const int r = (int)(grp / groups_per_row), g = (int)(grp % groups_per_row);
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
    const __nv_fp8_e4m3 scale_bits(fmaxf(amax / 6.f, 1.f / 512.f));
    const float scale = float(scale_bits);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t q0 = (uint32_t)__nv_cvt_float_to_fp4(v[2 * i] / scale, __NV_E2M1, cudaRoundNearest) & 0xFu;
        const uint32_t q1 = (uint32_t)__nv_cvt_float_to_fp4(v[2 * i + 1] / scale, __NV_E2M1, cudaRoundNearest) & 0xFu;
        const uint32_t byte = q0 | (q1 << 4);
        if (i < 4) lo |= byte << (8 * i);
        else hi |= byte << (8 * (i - 4));
    }
    *reinterpret_cast<uint2 *>(packed + grp * 8) = make_uint2(lo, hi);
    const size_t atom = ((size_t)(r / 128) * (groups_per_row / 4) + g / 4) * 512;
    sf[atom + (r % 32) * 16 + ((r % 128) / 32) * 4 + (g % 4)] = scale_bits.__x;
}

}  // namespace lb
}  // namespace mk

extern "C" int32_t mk_linear_batched_splits(int32_t n, int32_t k, int32_t sm_count) {
    // Enough (slab, split) items to give every SM work, while a split keeps at least 8 K blocks of 64.
    if (n <= 0 || k <= 0 || sm_count <= 0) return 1;
    const int slabs = (n + mk::lb::kSlabRows - 1) / mk::lb::kSlabRows, kblocks = k / mk::lb::kBlockK;
    int splits = 1;
    while (slabs * splits < sm_count && kblocks % (splits * 2) == 0 && kblocks / (splits * 2) >= 8) splits *= 2;
    return splits;
}

extern "C" int mk_linear_batched(const void *w_bf16, const void *x_bf16, void *y_bf16, float *partials, int32_t n, int32_t k,
                                 int32_t batch, int32_t splits, int32_t *error_word, void *stream) {
    return mk::lb::launch<false>(w_bf16, x_bf16, nullptr, nullptr, 1.0f, y_bf16, partials, n, k, batch, splits, error_word,
                                 (cudaStream_t)stream, "mk_linear_batched");
}

extern "C" int64_t mk_nvfp4_native_scale_bytes(int32_t rows, int32_t k) {
    if (rows <= 0 || k <= 0 || k % 64) return 0;
    return (int64_t)((rows + 127) / 128) * (k / 64) * 512;
}

extern "C" int mk_nvfp4_quantize_native(const void *input_bf16, void *packed, void *scales_native, int32_t rows, int32_t k,
                                        float tensor_scale, void *stream) {
    if (!input_bf16 || !packed || !scales_native || rows <= 0 || k <= 0 || (k % 64) != 0 || !(tensor_scale > 0.f)) {
        mk::set_last_error("mk_nvfp4_quantize_native: null pointer, k not a multiple of 64 or non-positive scale");
        return MK_ERR_BAD_ARGUMENT;
    }
    const long long groups = (long long)rows * (k / 16);
    const int threads = 256;
    return (int)mk::launch_pdl(mk::lb::quantize_native_kernel, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads), 0,
                               (cudaStream_t)stream, (const mk::bf16 *)input_bf16, (uint8_t *)packed, (uint8_t *)scales_native, rows, k,
                               tensor_scale);
}

extern "C" int mk_linear_batched_nvfp4(const void *w_packed, const void *w_scales_native, float w_tensor_scale, const void *x_packed,
                                       const void *x_scales_native, float x_tensor_scale, void *y_bf16, float *partials,
                                       int32_t n, int32_t k, int32_t batch, int32_t splits, int32_t *error_word, void *stream) {
    return mk::lb::launch<true>(w_packed, x_packed, (const uint8_t *)w_scales_native, (const uint8_t *)x_scales_native,
                                w_tensor_scale * x_tensor_scale, y_bf16, partials, n, k, batch, splits, error_word,
                                (cudaStream_t)stream, "mk_linear_batched_nvfp4");
}
