// Device-side building blocks shared by the decode megakernel and the
// standalone GEMV kernels: mbarrier / bulk-copy PTX wrappers, bounded waits,
// bf16 helpers.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mk {

using bf16 = __nv_bfloat16;

// ---------------------------------------------------------------------------
// shared-memory barriers and bulk copies
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Makes barrier initialisation visible to the bulk-copy (async proxy) engine.
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// Global -> shared bulk copy (TMA engine, untiled form).  Both addresses must
// be 16-byte aligned and `bytes` a multiple of 16.  Completion is signalled
// as transaction bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar,
                                          uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}

// Asks L2 to fetch `bytes` (multiple of 16) starting at a 16-byte aligned
// global address; nothing is written to shared memory and nothing signals
// completion.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src_gmem, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// Every lane of every participating warp must call this; the warp is
// reconverged first because lanes may arrive from a single-lane polling loop.
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    __syncwarp();
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------
// global-memory dependency counters
// ---------------------------------------------------------------------------

__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ int ld_relaxed_gpu(const int *p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Publishes every write that happens-before this call (the caller's own and,
// through a preceding warp/CTA barrier, its peers') to any thread that later
// acquires the counter.
__device__ __forceinline__ void red_release_gpu_add(int *p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// Only after fence_acq_rel_gpu() by the same thread: fence + relaxed add is a release.
__device__ __forceinline__ void red_relaxed_gpu_add(int *p, int v) {
    asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---------------------------------------------------------------------------
// tagged words: 32 bits of payload and a 32-bit launch tag in one 8-byte cell
// ---------------------------------------------------------------------------
// Activations that cross SMs inside a launch travel in 8-byte cells written and
// read with single 64-bit accesses.  A reader accepts a cell only if its tag is
// the current launch's, so payload and "it has been written" arrive together:
// no fence is needed between producing data and telling consumers about it.

__device__ __forceinline__ void st_tagged(unsigned long long *cell, uint32_t payload, uint32_t tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(cell), "l"(v) : "memory");
}

__device__ __forceinline__ ulonglong2 ld_tagged2(const unsigned long long *cell) {
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(cell) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long ld_tagged1(const unsigned long long *cell) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(cell) : "memory");
    return v;
}

// System-scope variants for cells that another GPU writes over NVLink.
__device__ __forceinline__ void st_tagged_sys(unsigned long long *cell, uint32_t payload, uint32_t tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | payload;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(cell), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long ld_tagged1_sys(const unsigned long long *cell) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(cell) : "memory");
    return v;
}

__device__ __forceinline__ bool tag_ok(unsigned long long v, uint32_t tag) { return (uint32_t)(v >> 32) == tag; }
__device__ __forceinline__ uint32_t tag_payload(unsigned long long v) { return (uint32_t)v; }

// ---------------------------------------------------------------------------
// bf16 helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

__device__ __forceinline__ void unpack8(const uint4 &v, float (&out)[8]) {
    out[0] = bf16_lo(v.x); out[1] = bf16_hi(v.x);
    out[2] = bf16_lo(v.y); out[3] = bf16_hi(v.y);
    out[4] = bf16_lo(v.z); out[5] = bf16_hi(v.z);
    out[6] = bf16_lo(v.w); out[7] = bf16_hi(v.w);
}

// Round-to-nearest-even through bf16 and back, the rounding every PyTorch
// bf16 op applies to its fp32 intermediate.
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float dot8(const uint4 &w, const float (&x)[8], float acc) {
    acc = fmaf(bf16_lo(w.x), x[0], acc); acc = fmaf(bf16_hi(w.x), x[1], acc);
    acc = fmaf(bf16_lo(w.y), x[2], acc); acc = fmaf(bf16_hi(w.y), x[3], acc);
    acc = fmaf(bf16_lo(w.z), x[4], acc); acc = fmaf(bf16_hi(w.z), x[5], acc);
    acc = fmaf(bf16_lo(w.w), x[6], acc); acc = fmaf(bf16_hi(w.w), x[7], acc);
    return acc;
}

__device__ __forceinline__ uint4 lds128(const void *p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr(p)));
    return v;
}

// Loads that bypass L1: activations are produced by other SMs during the same
// launch, and L1 is not coherent across SMs.
__device__ __forceinline__ float ldcg_bf16(const bf16 *p) {
    unsigned short raw = __ldcg(reinterpret_cast<const unsigned short *>(p));
    return __uint_as_float(static_cast<uint32_t>(raw) << 16);
}

__device__ __forceinline__ void ldcg8(const bf16 *p, float (&out)[8]) {
    uint4 v = __ldcg(reinterpret_cast<const uint4 *>(p));
    unpack8(v, out);
}

// Sum of 16 per-lane accumulators over the 32 lanes of a warp in 16 shuffles.
// On return lanes 2r and 2r+1 both hold the warp-wide total of acc[r].
__device__ __forceinline__ float warp_reduce16(float (&acc)[16], int lane) {
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int off = 16 >> step;      // 16, 8, 4, 2
        const int n = 8 >> step;         // 8, 4, 2, 1
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n; ++i) {
            float send = upper ? acc[i] : acc[i + n];
            float keep = upper ? acc[i + n] : acc[i];
            acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return acc[0] + __shfl_xor_sync(0xffffffffu, acc[0], 1);
}


// d += a x b for mma.sync.m16n8k16 (bf16 operands, fp32 accumulation) when rows 8..15
// of a - its fragments a1 and a3 - are zero.
__device__ __forceinline__ void mma_bf16_top(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// The same with the caller keeping only the top half of the accumulator: z0, z1 stand for rows 8..15,
// which stay zero and may be shared between any number of accumulators.
__device__ __forceinline__ void mma_bf16_top(float &d0, float &d1, float &z0, float &z1, uint32_t a0, uint32_t a2, uint32_t b0,
                                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d0), "+f"(d1), "+f"(z0), "+f"(z1)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-
// serialization attribute may start while its predecessor on the stream is still
// running.  pdl_launch_dependents() lets the successor start early; pdl_wait()
// returns once the predecessor has completed and its writes are visible (a no-op
// for a kernel launched without the attribute).  Everything a kernel reads from or
// writes to buffers that other kernels touch comes after pdl_wait().
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace mk
