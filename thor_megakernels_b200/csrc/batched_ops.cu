// The memory-bound operators of a batched decode step (16..128 sequences, each
// with its own cache length): embedding gather, residual add + RMSNorm,
// rotary embedding + KV append, decode attention over per-sequence cache
// lengths, SiLU-gate product, greedy argmax.  The dense contractions between
// them run on the tensor cores (linear_batched.cu).
//
// Arithmetic and bf16 rounding points are those of the reference's interpreter
// applied to every sequence on its own (megakernels/demos/latency/python_vm.py:
// RMSNorm :50-56, rotary + append :196-248, attention :277-346, SiLU product
// :146-165, residual add :59-80; the batched instruction set names the same
// steps, megakernels/demos/throughput/instructions.py:57-223).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "batched_ops.cuh"
#include "mk_device.cuh"

namespace mk {
namespace bo {

constexpr int kNormThreads = 256;
constexpr int kNormVecs = 8;   // float4 groups per thread: hidden sizes up to 8192

// LinOut (batched_ops.cuh) is the result of a batched linear as its consumers
// read it: bf16 y [batch, n], or the fp32 split-K partial sums [splits, batch, n],
// which are added here in split order, scaled and rounded to bf16 once - the
// value y would hold.
__device__ __forceinline__ float lin_value(const LinOut &o, int b, int i) {
    if (o.partials == nullptr) return __bfloat162float(o.y[(size_t)b * o.n + i]);
    float total = 0.f;
    for (int s = 0; s < o.splits; ++s) total += o.partials[((size_t)s * o.batch + b) * o.n + i];
    return round_bf16(total * o.scale);
}

// Two / four consecutive elements (i even / a multiple of 4): vector loads, the splits'
// loads independent of one another so that they are in flight together.
__device__ __forceinline__ float2 lin_value2(const LinOut &o, int b, int i) {
    if (o.partials == nullptr) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(o.y + (size_t)b * o.n + i));
    float2 total = make_float2(0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < o.splits; ++s) {
        const float2 v = *reinterpret_cast<const float2 *>(o.partials + ((size_t)s * o.batch + b) * o.n + i);
        total.x += v.x; total.y += v.y;
    }
    return make_float2(round_bf16(total.x * o.scale), round_bf16(total.y * o.scale));
}

__device__ __forceinline__ float4 load_bf16x4(const bf16 *p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store_bf16x4(bf16 *p, const float4 &v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t *>(&a);
    raw.y = *reinterpret_cast<const uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// sum of splits [s0, s1) for elements i..i+3, times the scale, rounded to bf16
__device__ __forceinline__ float4 partial_sum4(const LinOut &o, int b, int i, int s0, int s1) {
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = s0; s < s1; ++s) {
        const float4 v = *reinterpret_cast<const float4 *>(o.partials + ((size_t)s * o.batch + b) * o.n + i);
        total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
    }
    return make_float4(round_bf16(total.x * o.scale), round_bf16(total.y * o.scale), round_bf16(total.z * o.scale),
                       round_bf16(total.w * o.scale));
}
__device__ __forceinline__ float4 lin_value4(const LinOut &o, int b, int i) {
    if (o.partials == nullptr) return load_bf16x4(o.y + (size_t)b * o.n + i);
    return partial_sum4(o, b, i, 0, o.splits);
}

// hidden[b] = embed[token[b]]
__global__ void embed_kernel(const bf16 *__restrict__ embed, const int *__restrict__ tokens, bf16 *__restrict__ hidden,
                             int hidden_size, int vocab, int *__restrict__ error) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    // token ids come from device memory: one outside the table is clamped and reported (bit 1 of the error word)
    const int t = __ldg(tokens + b);
    const int tc = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
    if (tc != t && threadIdx.x == 0) atomicOr(error, 2);
    const uint4 *src = reinterpret_cast<const uint4 *>(embed + (size_t)tc * hidden_size);
    uint4 *dst = reinterpret_cast<uint4 *>(hidden + (size_t)b * hidden_size);
    for (int i = threadIdx.x; i < hidden_size / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// One CTA per sequence.  If a linear result is given (`add`), first the
// interpreter's residual add  hidden[b] = bf16(hidden[b] + bf16(linear[b])),
// then normed[b] = w * bf16(hidden[b] * rstd) with fp32 statistics.  `normed`
// may be null (residual update only).  With lin.group > 0 every `group`
// consecutive split-K partials form one addend that is rounded and added on
// its own: the down projection's 2048-column slices, which the interpreter adds
// one after the other (python_vm.py:59-80).
__global__ void __launch_bounds__(kNormThreads)
residual_norm_kernel(bf16 *__restrict__ hidden, const LinOut lin, int add, const bf16 *__restrict__ weight,
                     bf16 *__restrict__ normed, int hidden_size, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[kNormThreads / 32];
    const int b = blockIdx.x;
    const int vecs = hidden_size / 4;   // a thread owns elements 4v..4v+3 for v = tid, tid + 256, ... (at most kNormVecs of them)
    float4 h[kNormVecs];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kNormVecs; ++j) {
        const int v = threadIdx.x + j * kNormThreads;
        h[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v < vecs) {
            bf16 *hp = hidden + (size_t)b * hidden_size + 4 * v;
            float4 x = load_bf16x4(hp);
            if (add) {
                auto add_rounded = [&](const float4 &y) {
                    x = make_float4(round_bf16(x.x + y.x), round_bf16(x.y + y.y), round_bf16(x.z + y.z), round_bf16(x.w + y.w));
                };
                if (lin.partials != nullptr && lin.group > 0) {
                    for (int s0 = 0; s0 < lin.splits; s0 += lin.group) add_rounded(partial_sum4(lin, b, 4 * v, s0, s0 + lin.group));
                } else {
                    add_rounded(lin_value4(lin, b, 4 * v));
                }
                store_bf16x4(hp, x);
            }
            h[j] = x;
            ss = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, fmaf(x.w, x.w, ss))));
        }
    }
    if (normed == nullptr) return;
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += red[w];
    const float rstd = 1.0f / sqrtf(total / (float)hidden_size + eps);
#pragma unroll
    for (int j = 0; j < kNormVecs; ++j) {
        const int v = threadIdx.x + j * kNormThreads;
        if (v < vecs) {
            const float4 w = load_bf16x4(weight + 4 * v);
            store_bf16x4(normed + (size_t)b * hidden_size + 4 * v,
                         make_float4(w.x * round_bf16(h[j].x * rstd), w.y * round_bf16(h[j].y * rstd), w.z * round_bf16(h[j].z * rstd),
                                     w.w * round_bf16(h[j].w * rstd)));
        }
    }
}

// qkv [batch, (Hq + 2 Hkv) D] (bf16 linear output) -> q with rotary embedding,
// K (rotary) and V rows appended to the cache at each sequence's own position.
// The two elements (x0, x1) of a rotation pair become (x0 c0 - x1 s0, x1 c1 + x0 s1)
// in fp32 with separately rounded products and one bf16 rounding of the sum.
// half_split 0: pairs are adjacent elements (weights permuted for the
// "interleaved" tables, the latency instruction set); 1: element j of a head
// pairs with element j + D/2 (Hugging Face layout, the batched instruction set:
// megakernels/demos/throughput/python_vm.py:120-127).
__global__ void rope_append_kernel(const LinOut qkv, const int *__restrict__ pos_ids,
                                   const float *__restrict__ rope_cos, const float *__restrict__ rope_sin,
                                   bf16 *__restrict__ q_out, bf16 *__restrict__ k_cache, bf16 *__restrict__ v_cache,
                                   int layer, int batch, int kv_len, int hq, int hkv, int hd, int half_split, int slot_fixed) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int pos = __ldg(pos_ids + b);
    const int q_dim = hq * hd, kv_dim = hkv * hd, total = q_dim + 2 * kv_dim, half = hd / 2;
    // cache slot: the row's own (batched decode) or one slot for all rows (the rows are tokens of one prompt)
    const size_t cache_row = (((size_t)layer * batch + (slot_fixed >= 0 ? slot_fixed : b)) * kv_len + pos) * kv_dim;
    auto store2 = [&](int i, float y0, float y1) {   // elements i, i + 1 of the row (i even)
        const __nv_bfloat162 v = __floats2bfloat162_rn(y0, y1);
        if (i < q_dim) *reinterpret_cast<__nv_bfloat162 *>(q_out + (size_t)b * q_dim + i) = v;
        else if (i < q_dim + kv_dim) *reinterpret_cast<__nv_bfloat162 *>(k_cache + cache_row + (i - q_dim)) = v;
        else *reinterpret_cast<__nv_bfloat162 *>(v_cache + cache_row + (i - q_dim - kv_dim)) = v;
    };
    // a unit = two rotation pairs = two 2-element loads A and B:
    //   adjacent pairs: A = (i, i+1), B = (i+2, i+3), pairs (A.x, A.y), (B.x, B.y)
    //   half-split:     A = (i, i+1), B = (i+half, i+half+1), pairs (A.x, B.x), (A.y, B.y)
    for (int unit = threadIdx.x; unit < total / 4; unit += blockDim.x) {
        int ia, ib;
        if (half_split) {
            const int head = unit / (half / 2), j = 2 * (unit % (half / 2));
            ia = head * hd + j;
            ib = ia + half;
        } else {
            ia = 4 * unit;
            ib = ia + 2;
        }
        const float2 A = lin_value2(qkv, b, ia), B = lin_value2(qkv, b, ib);
        if (ia >= q_dim + kv_dim) {   // V: copied
            store2(ia, A.x, A.y);
            store2(ib, B.x, B.y);
            continue;
        }
        const int da = ia % hd, db = ib % hd;
        const float2 ca = *reinterpret_cast<const float2 *>(rope_cos + (size_t)pos * hd + da);
        const float2 sa = *reinterpret_cast<const float2 *>(rope_sin + (size_t)pos * hd + da);
        const float2 cb = *reinterpret_cast<const float2 *>(rope_cos + (size_t)pos * hd + db);
        const float2 sb = *reinterpret_cast<const float2 *>(rope_sin + (size_t)pos * hd + db);
        auto rot0 = [](float x0, float x1, float c, float s_) { return round_bf16(__fadd_rn(__fmul_rn(x0, c), __fmul_rn(-x1, s_))); };
        auto rot1 = [](float x0, float x1, float c, float s_) { return round_bf16(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s_))); };
        if (half_split) {   // pairs (A.x, B.x) and (A.y, B.y); first elements use the tables at da, second at db
            store2(ia, rot0(A.x, B.x, ca.x, sa.x), rot0(A.y, B.y, ca.y, sa.y));
            store2(ib, rot1(A.x, B.x, cb.x, sb.x), rot1(A.y, B.y, cb.y, sb.y));
        } else {            // pairs (A.x, A.y) and (B.x, B.y)
            store2(ia, rot0(A.x, A.y, ca.x, sa.x), rot1(A.x, A.y, ca.y, sa.y));
            store2(ib, rot0(B.x, B.y, cb.x, sb.x), rot1(B.x, B.y, cb.y, sb.y));
        }
    }
}

// Decode attention of one (sequence, KV head, cache split): the 4 query heads of
// the group over a contiguous share of cache rows 0..pos (the row appended by this
// step included), on the tensor cores.
//
// Data movement: the share's rows go through a shared-memory pipeline (4 stages of
// 64 rows for 64-wide heads, 3 for 128-wide ones) filled with 16-byte asynchronous
// copies by all 128 threads; several CTAs are resident per SM, which keeps tens of
// KiB per SM in flight - at large batch the cache, not the weights, is most of a
// step's bytes.  16-byte chunk c of row r sits at chunk c ^ (r % 8) of its row, so
// the 8 rows an ldmatrix phase touches fall into different banks.
//
// Arithmetic: warp w owns rows 16w..16w+15 of every stage.  Scores are
// mma.sync.m16n8k16 with the query heads as M (4 real rows, the rest zero), the
// cache rows as N and the head dimension as K; K fragments come from ldmatrix.
// The fp32 score fragment of a thread - head lane/4, rows 2t, 2t+1, 8+2t, 9+2t -
// is exactly the A fragment of the second product (probabilities x V, V through
// ldmatrix.trans), so probabilities go from registers to the tensor cores after an
// online-softmax update (running max in log2 units, rescaled sums).  Scores,
// softmax and sums are fp32; a probability enters the second product as two bf16
// terms (value + remainder), which keeps about 16 of its significant bits.
//
// splits == 1: the merged result leaves as bf16 attention output.  Otherwise each
// split writes its unnormalised state (max in log2 units, sum, output) to
// `partial` [batch, Hq, splits, D + 2] and attention_merge_kernel combines them.
constexpr int kAttnWarps = 4;
constexpr int kAttnRows = 64;   // cache rows per stage: 16 per warp

template <int D>
struct AttnShape {
    static constexpr int kStages = D == 64 ? 4 : 3;
    static constexpr int kRowBytes = D * 2, kChunksPerRow = D / 8;
    static constexpr int kStageBytes = kAttnRows * kRowBytes;   // per K (and per V)
    static constexpr int kPartFloats = kAttnWarps * 4 * (D + 2);
    static constexpr size_t kSmemBytes = (size_t)2 * kStages * kStageBytes + kPartFloats * sizeof(float);
};

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <int D>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_batched_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ k_cache, const bf16 *__restrict__ v_cache,
                         const int *__restrict__ pos_ids, bf16 *__restrict__ out, float *__restrict__ partial, int splits,
                         int layer, int cache_batch, int kv_len, int hq, int hkv, float attn_scale, int slot_fixed) {
    pdl_launch_dependents();
    pdl_wait();
    using S = AttnShape<D>;
    extern __shared__ __align__(128) uint8_t attn_smem[];
    uint8_t *stage_k = attn_smem, *stage_v = attn_smem + S::kStages * S::kStageBytes;
    float(*part)[4][D + 2] = reinterpret_cast<float(*)[4][D + 2]>(attn_smem + 2 * S::kStages * S::kStageBytes);
    const int kv_head = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int seq_len = __ldg(pos_ids + b) + 1;
    // this split's share of the rows, in whole stages
    const int stages_total = (seq_len + kAttnRows - 1) / kAttnRows;
    const int per_split = (stages_total + splits - 1) / splits;
    const int t_begin = min(split * per_split, stages_total) * kAttnRows;
    const int t_end = min(min((split + 1) * per_split, stages_total) * kAttnRows, seq_len);
    const int n_stages = t_end > t_begin ? (t_end - t_begin + kAttnRows - 1) / kAttnRows : 0;
    const size_t tok_stride = (size_t)hkv * D;
    const size_t base = (((size_t)layer * cache_batch + (slot_fixed >= 0 ? slot_fixed : b)) * kv_len) * tok_stride + (size_t)kv_head * D;
    const uint8_t *kbase = reinterpret_cast<const uint8_t *>(k_cache + base), *vbase = reinterpret_cast<const uint8_t *>(v_cache + base);
    const uint32_t sk = smem_addr(stage_k), sv = smem_addr(stage_v);

    auto fill = [&](int st_idx) {
        const int slot = st_idx % S::kStages, t0 = t_begin + st_idx * kAttnRows;
        for (int c = threadIdx.x; c < kAttnRows * S::kChunksPerRow; c += kAttnWarps * 32) {
            const int r = c / S::kChunksPerRow, ch = c % S::kChunksPerRow;
            const uint32_t off = slot * S::kStageBytes + r * S::kRowBytes + ((ch ^ (r & 7)) << 4);
            if (t0 + r < t_end) {
                const size_t src = (size_t)(t0 + r) * tok_stride * 2 + ch * 16;
                cp_async16(sk + off, kbase + src);
                cp_async16(sv + off, vbase + src);
            } else {  // rows past the share: zeros, so that they add nothing (and no NaN) to either product
                *reinterpret_cast<uint4 *>(stage_k + off) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(stage_v + off) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // prologue: stages 0 .. kStages-2 in flight (empty groups keep the counting uniform)
    for (int i = 0; i < S::kStages - 1; ++i) {
        if (i < n_stages) fill(i);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // query fragments: head g (lanes with g < 4), dimensions 16 ks + {2t, 2t+1} and + 8
    uint32_t qa[D / 16][2];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        qa[ks][0] = qa[ks][1] = 0u;
        if (g < 4) {
            const bf16 *qp = q + (size_t)b * hq * D + (size_t)(kv_head * 4 + g) * D + ks * 16 + 2 * t;
            qa[ks][0] = *reinterpret_cast<const uint32_t *>(qp);
            qa[ks][1] = *reinterpret_cast<const uint32_t *>(qp + 8);
        }
    }
    float m = -INFINITY, l = 0.f;
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const float scale_log2e = attn_scale * 1.4426950408889634f;
    const int r0 = warp * 16;                 // this warp's rows within a stage
    const int lrow = lane & 7, lmat = lane >> 3;  // ldmatrix: this lane addresses row lrow of matrix lmat

    for (int st_idx = 0; st_idx < n_stages; ++st_idx) {
        asm volatile("cp.async.wait_group %0;" ::"n"(S::kStages - 2) : "memory");  // stage st_idx has landed (for this thread)
        __syncthreads();                                                           // ... and for everybody; stage st_idx-1 is free
        if (st_idx + S::kStages - 1 < n_stages) fill(st_idx + S::kStages - 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int slot = st_idx % S::kStages, t0 = t_begin + st_idx * kAttnRows;
        const int rows = t_end - t0;          // valid rows of this stage (may exceed 64)
        if (r0 >= rows) continue;             // warp-uniform: nothing of this stage belongs to the warp
        const uint32_t kb = sk + slot * S::kStageBytes, vb = sv + slot * S::kStageBytes;

        // scores[head][row]: two 8-row tiles, K dimension = head dimension
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
            const int r = r0 + nt * 8 + lrow;
#pragma unroll
            for (int k2 = 0; k2 < D / 32; ++k2) {   // one ldmatrix.x4 = chunks 4 k2 .. 4 k2 + 3 = two K steps
                uint32_t kf[4];
                ldmatrix_x4(kb + r * S::kRowBytes + (((4 * k2 + lmat) ^ (r & 7)) << 4), kf);
                mma_bf16_top(sc[nt], qa[2 * k2][0], qa[2 * k2][1], kf[0], kf[1]);
                mma_bf16_top(sc[nt], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], kf[2], kf[3]);
            }
        }
        // online softmax for head g over rows r0 + {2t, 2t+1, 8+2t, 9+2t}
        float sv4[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                sv4[2 * nt + e] = (r0 + nt * 8 + 2 * t + e < rows) ? sc[nt][e] * scale_log2e : -INFINITY;
        float mx = fmaxf(fmaxf(sv4[0], sv4[1]), fmaxf(sv4[2], sv4[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m, mx);                                    // finite: the warp has at least one valid row
        const float corr = (m == -INFINITY) ? 0.f : exp2f(m - mn);
        float pr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pr[i] = (g < 4 && sv4[i] > -INFINITY) ? exp2f(sv4[i] - mn) : 0.f;
        l = l * corr + (pr[0] + pr[1]) + (pr[2] + pr[3]);
        m = mn;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr; o[i][1] *= corr; }
        // The tensor core takes bf16 operands; a probability goes in as the sum of two bf16
        // values (the rounded value and the rounded remainder, about 16 significant bits), so
        // the weighted sum keeps fp32-like accuracy at the cost of a second MMA per tile.
        uint32_t pa_hi[2], pa_lo[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const __nv_bfloat162 hi = __floats2bfloat162_rn(pr[2 * i], pr[2 * i + 1]);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(pr[2 * i] - __low2float(hi), pr[2 * i + 1] - __high2float(hi));
            pa_hi[i] = *reinterpret_cast<const uint32_t *>(&hi);
            pa_lo[i] = *reinterpret_cast<const uint32_t *>(&lo);
        }
        // out[head][d] += p[head][row] * V[row][d]: 16 rows as K, 8 dimensions per tile, two tiles per ldmatrix
#pragma unroll
        for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t vf[4];
            const int r = r0 + (lmat & 1) * 8 + lrow;
            ldmatrix_x4_trans(vb + r * S::kRowBytes + (((2 * d2 + (lmat >> 1)) ^ (r & 7)) << 4), vf);
            mma_bf16_top(o[2 * d2], pa_hi[0], pa_hi[1], vf[0], vf[1]);
            mma_bf16_top(o[2 * d2], pa_lo[0], pa_lo[1], vf[0], vf[1]);
            mma_bf16_top(o[2 * d2 + 1], pa_hi[0], pa_hi[1], vf[2], vf[3]);
            mma_bf16_top(o[2 * d2 + 1], pa_lo[0], pa_lo[1], vf[2], vf[3]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (g < 4) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            part[warp][g][i * 8 + 2 * t] = o[i][0];
            part[warp][g][i * 8 + 2 * t + 1] = o[i][1];
        }
        if (t == 0) {
            part[warp][g][D] = m;
            part[warp][g][D + 1] = l;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 4 * D; idx += kAttnWarps * 32) {
        const int hh = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, part[w][hh][D]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = part[w][hh][D];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            L = fmaf(part[w][hh][D + 1], f, L);
            O = fmaf(part[w][hh][d], f, O);
        }
        const int head = kv_head * 4 + hh;
        if (splits == 1) {
            out[(size_t)b * hq * D + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            float *dst = partial + (((size_t)b * hq + head) * splits + split) * (D + 2);
            dst[d] = O;
            if (d == 0) {
                dst[D] = M;
                dst[D + 1] = L;
            }
        }
    }
}

// Combines the splits of one (sequence, query head): weights exp2(m_s - max m), one thread per head dimension.
__global__ void attention_merge_kernel(const float *__restrict__ partial, bf16 *__restrict__ out, int splits, int hq, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float *src = partial + (((size_t)b * hq + head) * splits) * (D + 2);
    float M = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, src[sp * (D + 2) + D]);
    float L = 0.f, O = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
        const float ms = src[sp * (D + 2) + D];
        const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        L = fmaf(src[sp * (D + 2) + D + 1], f, L);
        O = fmaf(src[sp * (D + 2) + d], f, O);
    }
    out[(size_t)b * hq * D + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

// act[b, i] = bf16(bf16(silu(gate[b, i])) * up[b, i]) from the two linears'
// results (an `up` without buffers counts as 1: SiLU only).  With `round_silu` 0 the product is rounded once (the rule of the
// reference's quantised model, tools/analysis/nvfp4/model_reference.py:39-61).
__global__ void silu_mul_kernel(const LinOut up, const LinOut gate, bf16 *__restrict__ act, int batch, int inter, int round_silu) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total4 = (size_t)batch * inter / 4;   // four consecutive elements per thread and iteration
    const bool no_up = up.y == nullptr && up.partials == nullptr;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(4 * idx / inter), i = (int)(4 * idx % inter);
        const float4 g = lin_value4(gate, b, i);
        const float4 u = no_up ? make_float4(1.f, 1.f, 1.f, 1.f) : lin_value4(up, b, i);
        auto f = [&](float gv, float uv) {
            float a = gv / (1.0f + expf(-gv));
            if (round_silu) a = round_bf16(a);
            return a * uv;
        };
        store_bf16x4(act + 4 * idx, make_float4(f(g.x, u.x), f(g.y, u.y), f(g.z, u.z), f(g.w, u.w)));
    }
}

// token[b] = argmax_i logits[b, i], lowest index on ties.  One CTA per sequence.
constexpr int kArgmaxThreads = 1024;
__global__ void __launch_bounds__(kArgmaxThreads) argmax_kernel(const bf16 *__restrict__ logits, int *__restrict__ tokens, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned long long best_s[kArgmaxThreads / 32];
    const int b = blockIdx.x;
    const bf16 *row = logits + (size_t)b * vocab;
    unsigned long long best = 0ull;
    auto consider = [&](uint32_t bits, int i) {
        bits = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);  // order-preserving
        const unsigned long long key = ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
        if (key > best) best = key;
    };
    // 16-byte loads (8 logits) while the row allows it, the remainder one by one
    const int vec_end = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) ? (vocab / 8) * 8 : 0;
#pragma unroll 4
    for (int i = 8 * threadIdx.x; i < vec_end; i += 8 * kArgmaxThreads) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(row + i));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            consider(w[j] & 0xffffu, i + 2 * j);
            consider(w[j] >> 16, i + 2 * j + 1);
        }
    }
    for (int i = vec_end + threadIdx.x; i < vocab; i += kArgmaxThreads) consider((uint32_t)__bfloat16_as_ushort(row[i]), i);
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
        if (o > best) best = o;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kArgmaxThreads / 32; ++w)
            if (best_s[w] > best) best = best_s[w];
        tokens[b] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
    }
}

}  // namespace bo

// launchers used by the batched step (batched_step.cu); declared in batched_ops.cuh
cudaError_t launch_embed(const bf16 *embed, const int *tokens, bf16 *hidden, int batch, int hidden_size, int vocab, int *error,
                         cudaStream_t st) {
    return launch_pdl(bo::embed_kernel, dim3(batch), dim3(128), 0, st, embed, tokens, hidden, hidden_size, vocab, error);
}

cudaError_t launch_residual_norm(bf16 *hidden, const bo::LinOut &lin, int add, const bf16 *weight, bf16 *normed, int batch,
                                 int hidden_size, float eps, cudaStream_t st) {
    if (hidden_size % 4 || hidden_size > 4 * bo::kNormThreads * bo::kNormVecs) return cudaErrorInvalidValue;
    return launch_pdl(bo::residual_norm_kernel, dim3(batch), dim3(bo::kNormThreads), 0, st, hidden, lin, add, weight, normed, hidden_size,
                      eps);
}

cudaError_t launch_rope_append(const bo::LinOut &qkv, const int *pos_ids, const float *rope_cos, const float *rope_sin, bf16 *q_out,
                               bf16 *k_cache, bf16 *v_cache, int layer, int rows, int cache_batch, int kv_len, int hq, int hkv,
                               int hd, int half_split, int slot_fixed, cudaStream_t st) {
    return launch_pdl(bo::rope_append_kernel, dim3(rows), dim3(256), 0, st, qkv, pos_ids, rope_cos, rope_sin, q_out, k_cache, v_cache,
                      layer, cache_batch, kv_len, hq, hkv, hd, half_split, slot_fixed);
}

namespace bo {

// dst[i] = value + i * step
__global__ void fill_int_kernel(int *__restrict__ dst, int value, int step, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value + i * step;
}

// Positions arrive in device memory, where the host cannot look at them.  They are copied
// into the handle's own array, clamped into [0, limit), so that no later kernel indexes
// outside the rotary tables or the cache; a value that had to be clamped sets bit 1 of the
// error word.
__global__ void sanitize_positions_kernel(const int *__restrict__ pos_ids, int *__restrict__ pos_out, int batch, int pos_limit,
                                          int *__restrict__ error) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    const int q = pos_ids[b];
    const int qc = q < 0 ? 0 : (q >= pos_limit ? pos_limit - 1 : q);
    pos_out[b] = qc;
    if (qc != q) atomicOr(error, 2);
}

// Final values of the batched instruction set's dependency counters
// (megakernels/demos/throughput/python_vm.py: each solver's closing update) for
// the operators a schedule covers.  barriers [layers, 10, batch, cols]; row
// index = 128-sequence block.  One CTA per (layer, opcode - 1); covered[layer]
// has bit (opcode - 1) set for covered operators.
__global__ void barrier_fill_kernel(int *__restrict__ barriers, const int *__restrict__ covered, int batch, int cols,
                                    int batch_blocks, int hq, int hkv, int out_blocks, int inter_blocks) {
    pdl_launch_dependents();
    pdl_wait();
    const int layer = blockIdx.x / 10, op = blockIdx.x % 10;  // op = opcode - 1
    if (!((covered[layer] >> op) & 1)) return;
    int *base = barriers + ((size_t)layer * 10 + op) * batch * cols;
    int width = 1, value = 0;
    switch (op) {
        case 0: case 4: case 8: value = 128; break;                 // norms: one count per sequence of the block
        case 1: width = hq + 2 * hkv; value = 1; break;             // one flag per head of the QKV row
        case 2: value = 128 * hkv; break;                           // attention: per sequence and KV head
        case 3: case 7: value = out_blocks; break;                  // o_proj / down_proj output blocks
        case 5: width = inter_blocks; value = 1; break;             // gate blocks
        case 6: value = inter_blocks; break;                        // up blocks
        default: return;                                            // LM head publishes nothing
    }
    for (int i = threadIdx.x; i < batch_blocks * width; i += blockDim.x) base[(size_t)(i / width) * cols + i % width] = value;
}

}  // namespace bo

cudaError_t launch_sanitize_positions(const int *pos_ids, int *pos_out, int batch, int pos_limit, int *error, cudaStream_t st) {
    return launch_pdl(bo::sanitize_positions_kernel, dim3((batch + 127) / 128), dim3(128), 0, st, pos_ids, pos_out, batch, pos_limit,
                      error);
}

cudaError_t launch_fill_int(int *dst, int value, int step, int n, cudaStream_t st) {
    return launch_pdl(bo::fill_int_kernel, dim3((n + 255) / 256), dim3(256), 0, st, dst, value, step, n);
}

cudaError_t launch_barrier_fill(int *barriers, const int *covered, int layers, int batch, int cols, int batch_blocks, int hq,
                                int hkv, int out_blocks, int inter_blocks, cudaStream_t st) {
    return launch_pdl(bo::barrier_fill_kernel, dim3(layers * 10), dim3(128), 0, st, barriers, covered, batch, cols, batch_blocks, hq, hkv,
                      out_blocks, inter_blocks);
}

// Cache splits per (sequence, KV head): enough CTAs to fill the GPU a few times over at small
// batch, none at large batch; at most `max_splits` (what the caller's partial buffer holds).
int attention_batched_splits(int batch, int hkv, int sms, int max_splits) {
    // 8 CTAs' worth of work per SM: with three CTAs resident per SM and cache lengths that differ by up to 8x
    // between sequences, smaller shares even out the last wave
    int splits = 1;
    while (batch * hkv * splits < 8 * sms && splits * 2 <= max_splits) splits *= 2;
    return splits;
}

template <int D>
static cudaError_t launch_attention_d(dim3 grid, cudaStream_t st, const bf16 *q, const bf16 *k_cache, const bf16 *v_cache, const int *pos_ids,
                                      bf16 *out, float *partial, int splits, int layer, int cache_batch, int kv_len, int hq, int hkv,
                                      float attn_scale, int slot_fixed) {
    static bool configured[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 64 && !configured[device]) {
        e = cudaFuncSetAttribute(bo::attention_batched_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)bo::AttnShape<D>::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[device] = true;
    }
    return launch_pdl(bo::attention_batched_kernel<D>, grid, dim3(bo::kAttnWarps * 32), bo::AttnShape<D>::kSmemBytes, st, q, k_cache,
                      v_cache, pos_ids, out, partial, splits, layer, cache_batch, kv_len, hq, hkv, attn_scale, slot_fixed);
}

cudaError_t launch_attention_batched(const bf16 *q, const bf16 *k_cache, const bf16 *v_cache, const int *pos_ids, bf16 *out,
                                     float *partial, int splits, int layer, int batch, int cache_batch, int kv_len, int hq, int hkv,
                                     int hd, float attn_scale, int slot_fixed, cudaStream_t st) {
    const dim3 grid(hkv, batch, splits);
    cudaError_t e = hd == 64 ? launch_attention_d<64>(grid, st, q, k_cache, v_cache, pos_ids, out, partial, splits, layer, cache_batch,
                                                      kv_len, hq, hkv, attn_scale, slot_fixed)
                             : launch_attention_d<128>(grid, st, q, k_cache, v_cache, pos_ids, out, partial, splits, layer, cache_batch,
                                                       kv_len, hq, hkv, attn_scale, slot_fixed);
    if (e != cudaSuccess || splits == 1) return e;
    return launch_pdl(bo::attention_merge_kernel, dim3(hq, batch), dim3(hd), 0, st, partial, out, splits, hq, hd);
}

cudaError_t launch_silu_mul(const bo::LinOut &up, const bo::LinOut &gate, bf16 *act, int batch, int inter, int round_silu,
                            cudaStream_t st) {
    const size_t total = (size_t)batch * inter / 4;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    return launch_pdl(bo::silu_mul_kernel, dim3(blocks), dim3(256), 0, st, up, gate, act, batch, inter, round_silu);
}

cudaError_t launch_argmax(const bf16 *logits, int *tokens, int batch, int vocab, cudaStream_t st) {
    return launch_pdl(bo::argmax_kernel, dim3(batch), dim3(bo::kArgmaxThreads), 0, st, logits, tokens, vocab);
}

static bool g_launch_overlap = true;
bool launch_overlap_enabled() { return g_launch_overlap; }

}  // namespace mk

// 1 (default): the batched path's kernels are launched with the programmatic-stream-
// serialization attribute; 0: plain stream order.  Results do not change.
extern "C" int mk_batched_set_overlap(int32_t enabled) {
    mk::g_launch_overlap = enabled != 0;
    return 0;
}
