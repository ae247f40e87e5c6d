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

// hidden[b] = embed[token[b]]
__global__ void embed_kernel(const bf16 *__restrict__ embed, const int *__restrict__ tokens, bf16 *__restrict__ hidden,
                             int hidden_size) {
    const int b = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(embed + (size_t)__ldg(tokens + b) * hidden_size);
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
    extern __shared__ float row[];  // hidden_size floats
    __shared__ float red[kNormThreads / 32];
    const int b = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden_size; i += kNormThreads) {
        float h = __bfloat162float(hidden[(size_t)b * hidden_size + i]);
        if (add) {
            if (lin.partials != nullptr && lin.group > 0) {
                for (int s0 = 0; s0 < lin.splits; s0 += lin.group) {
                    float total = 0.f;
                    for (int sp = s0; sp < s0 + lin.group; ++sp) total += lin.partials[((size_t)sp * lin.batch + b) * lin.n + i];
                    h = round_bf16(h + round_bf16(total * lin.scale));
                }
            } else {
                h = round_bf16(h + lin_value(lin, b, i));
            }
            hidden[(size_t)b * hidden_size + i] = __float2bfloat16_rn(h);
        }
        row[i] = h;
        ss = fmaf(h, h, ss);
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
    for (int i = threadIdx.x; i < hidden_size; i += kNormThreads) {
        const float w = __bfloat162float(weight[i]);
        normed[(size_t)b * hidden_size + i] = __float2bfloat16_rn(w * round_bf16(row[i] * rstd));
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
    const int b = blockIdx.x;
    const int pos = __ldg(pos_ids + b);
    const int q_dim = hq * hd, kv_dim = hkv * hd, total = q_dim + 2 * kv_dim;
    // cache slot: the row's own (batched decode) or one slot for all rows (the rows are tokens of one prompt)
    const size_t cache_row = (((size_t)layer * batch + (slot_fixed >= 0 ? slot_fixed : b)) * kv_len + pos) * kv_dim;
    auto store = [&](int i, float y) {
        const bf16 v = __float2bfloat16_rn(y);
        if (i < q_dim) q_out[(size_t)b * q_dim + i] = v;
        else if (i < q_dim + kv_dim) k_cache[cache_row + (i - q_dim)] = v;
        else v_cache[cache_row + (i - q_dim - kv_dim)] = v;
    };
    for (int pair = threadIdx.x; pair < total / 2; pair += blockDim.x) {
        const int half = hd / 2;
        const int i0 = half_split ? (pair / half) * hd + pair % half : 2 * pair;
        const int i1 = half_split ? i0 + half : i0 + 1;
        const float x0 = lin_value(qkv, b, i0), x1 = lin_value(qkv, b, i1);
        float y0 = x0, y1 = x1;
        if (i0 < q_dim + kv_dim) {
            const int d0 = i0 % hd, d1 = i1 % hd;
            const float c0 = __ldg(rope_cos + (size_t)pos * hd + d0), s0 = __ldg(rope_sin + (size_t)pos * hd + d0);
            const float c1 = __ldg(rope_cos + (size_t)pos * hd + d1), s1 = __ldg(rope_sin + (size_t)pos * hd + d1);
            y0 = round_bf16(__fadd_rn(__fmul_rn(x0, c0), __fmul_rn(-x1, s0)));
            y1 = round_bf16(__fadd_rn(__fmul_rn(x1, c1), __fmul_rn(x0, s1)));
        }
        if (!half_split) {
            const __nv_bfloat162 out = __floats2bfloat162_rn(y0, y1);
            if (i0 < q_dim) *reinterpret_cast<__nv_bfloat162 *>(q_out + (size_t)b * q_dim + i0) = out;
            else if (i0 < q_dim + kv_dim) *reinterpret_cast<__nv_bfloat162 *>(k_cache + cache_row + (i0 - q_dim)) = out;
            else *reinterpret_cast<__nv_bfloat162 *>(v_cache + cache_row + (i0 - q_dim - kv_dim)) = out;
        } else {
            store(i0, y0);
            store(i1, y1);
        }
    }
}

// Decode attention of one (sequence, KV head, cache split): the 4 query heads of
// the group over a contiguous share of cache rows 0..pos (the row appended by this
// step included).  fp32 scores, softmax and weighted sum.
//
// The cache rows of the share go through a 4-stage shared-memory pipeline filled
// with 16-byte asynchronous copies (cp.async) by all 128 threads: every lane moves
// a different 16 bytes, three stages are in flight while the fourth is consumed,
// and several CTAs are resident per SM - that is what keeps HBM busy here; at
// large batch the cache, not the weights, is most of a step's bytes.  A warp takes
// rows w, w+4, ... of a stage; lane (h = lane/8, sub = lane%8) owns query head h
// and DPL = D/8 head dimensions and reads its part of a row from shared memory.
//
// splits == 1: the merged result leaves as bf16 attention output.  Otherwise each
// split writes its unnormalised state (max in log2 units, sum, output) to
// `partial` [batch, Hq, splits, D + 2] and attention_merge_kernel combines them.
constexpr int kAttnWarps = 4;
constexpr int kAttnStages = 4;
// cache rows per stage: 32 for 64-wide heads, 16 for 128-wide ones (8 KiB of K + V per stage either way)

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}

template <int DPL>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_batched_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ k_cache, const bf16 *__restrict__ v_cache,
                         const int *__restrict__ pos_ids, bf16 *__restrict__ out, float *__restrict__ partial, int splits,
                         int layer, int cache_batch, int kv_len, int hq, int hkv, float attn_scale, int slot_fixed) {
    constexpr int V = DPL / 8, D = DPL * 8;
    constexpr int kAttnRows = DPL == 8 ? 32 : 16;
    constexpr int kRowBytes = D * 2, kStageBytes = kAttnRows * kRowBytes;  // per K (and per V)
    __shared__ __align__(16) uint8_t stage_k[kAttnStages][kStageBytes];
    __shared__ __align__(16) uint8_t stage_v[kAttnStages][kStageBytes];
    __shared__ float part[kAttnWarps][4][D + 2];
    const int kv_head = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = lane >> 3, sub = lane & 7, d0 = sub * DPL;
    const int seq_len = __ldg(pos_ids + b) + 1;
    // this split's share of the rows, in whole stages
    const int stages_total = (seq_len + kAttnRows - 1) / kAttnRows;
    const int per_split = (stages_total + splits - 1) / splits;
    const int t_begin = min(split * per_split, stages_total) * kAttnRows;
    const int t_end = min(min((split + 1) * per_split, stages_total) * kAttnRows, seq_len);
    const int n_stages = t_end > t_begin ? (t_end - t_begin + kAttnRows - 1) / kAttnRows : 0;
    const size_t tok_stride = (size_t)hkv * D;
    const size_t base = (((size_t)layer * cache_batch + (slot_fixed >= 0 ? slot_fixed : b)) * kv_len) * tok_stride + (size_t)kv_head * D;
    const bf16 *kbase = k_cache + base, *vbase = v_cache + base;

    // one stage = kAttnRows rows of K and of V; chunk c of 16 bytes: row c / (kRowBytes/16), offset c % ...
    constexpr int kChunksPerRow = kRowBytes / 16, kChunks = kAttnRows * kChunksPerRow;
    auto fill = [&](int st_idx) {
        const int slot = st_idx % kAttnStages, t0 = t_begin + st_idx * kAttnRows;
        for (int c = threadIdx.x; c < kChunks; c += kAttnWarps * 32) {
            const int r = c / kChunksPerRow, o = (c % kChunksPerRow) * 16;
            if (t0 + r < t_end) {
                cp_async16(&stage_k[slot][r * kRowBytes + o], reinterpret_cast<const uint8_t *>(kbase + (size_t)(t0 + r) * tok_stride) + o);
                cp_async16(&stage_v[slot][r * kRowBytes + o], reinterpret_cast<const uint8_t *>(vbase + (size_t)(t0 + r) * tok_stride) + o);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // prologue: stages 0 .. kAttnStages-2 in flight (empty groups keep the counting uniform)
    for (int i = 0; i < kAttnStages - 1; ++i) {
        if (i < n_stages) fill(i);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }

    float qf[DPL];
    {
        const bf16 *qp = q + (size_t)b * hq * D + (size_t)(kv_head * 4 + h) * D + d0;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float tmp[8];
            unpack8(*reinterpret_cast<const uint4 *>(qp + 8 * v), tmp);
#pragma unroll
            for (int i = 0; i < 8; ++i) qf[8 * v + i] = tmp[i];
        }
    }
    float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    const float scale_log2e = attn_scale * 1.4426950408889634f;

    for (int st_idx = 0; st_idx < n_stages; ++st_idx) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kAttnStages - 2) : "memory");  // stage st_idx has landed (for this thread)
        __syncthreads();                                                              // ... and for everybody; stage st_idx-1 is free
        if (st_idx + kAttnStages - 1 < n_stages) fill(st_idx + kAttnStages - 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int slot = st_idx % kAttnStages, t0 = t_begin + st_idx * kAttnRows;
        const int rows = min(kAttnRows, t_end - t0);
        // a warp's rows of this stage: w, w+4, ...; all scores first, one running-max update, then the sums
        constexpr int kPerWarp = kAttnRows / kAttnWarps;
        float sc[kPerWarp];
#pragma unroll
        for (int j = 0; j < kPerWarp; ++j) {
            const int r = warp + j * kAttnWarps;
            float d = 0.f;
            if (r < rows) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    float kf[8];
                    unpack8(*reinterpret_cast<const uint4 *>(&stage_k[slot][r * kRowBytes + d0 * 2 + 16 * v]), kf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) d = fmaf(qf[8 * v + i], kf[i], d);
                }
            }
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            sc[j] = r < rows ? d * scale_log2e : -INFINITY;
        }
        float mn = m;
#pragma unroll
        for (int j = 0; j < kPerWarp; ++j) mn = fmaxf(mn, sc[j]);
        if (mn > -INFINITY) {   // this warp has at least one row so far
            const float corr = exp2f(m - mn);  // exp2(-inf) = 0 the first time
            l *= corr;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] *= corr;
#pragma unroll
            for (int j = 0; j < kPerWarp; ++j) {
                const int r = warp + j * kAttnWarps;
                if (r < rows) {
                    const float pr = exp2f(sc[j] - mn);
                    l += pr;
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        float vf[8];
                        unpack8(*reinterpret_cast<const uint4 *>(&stage_v[slot][r * kRowBytes + d0 * 2 + 16 * v]), vf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[8 * v + i] = fmaf(pr, vf[i], acc[8 * v + i]);
                    }
                }
            }
            m = mn;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < DPL; ++i) part[warp][h][d0 + i] = acc[i];
    if (sub == 0) {
        part[warp][h][D] = m;
        part[warp][h][D + 1] = l;
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
    const size_t total = (size_t)batch * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(idx / inter), i = (int)(idx % inter);
        const float g = lin_value(gate, b, i);
        const float u = (up.y == nullptr && up.partials == nullptr) ? 1.0f : lin_value(up, b, i);
        float a = g / (1.0f + expf(-g));
        if (round_silu) a = round_bf16(a);
        act[idx] = __float2bfloat16_rn(a * u);
    }
}

// token[b] = argmax_i logits[b, i], lowest index on ties.  One CTA per sequence.
__global__ void __launch_bounds__(256) argmax_kernel(const bf16 *__restrict__ logits, int *__restrict__ tokens, int vocab) {
    __shared__ unsigned long long best_s[8];
    const int b = blockIdx.x;
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < vocab; i += 256) {
        uint32_t bits = (uint32_t)__bfloat16_as_ushort(logits[(size_t)b * vocab + i]);
        bits = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);  // order-preserving
        const unsigned long long key = ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
        if (key > best) best = key;
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
        if (o > best) best = o;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (best_s[w] > best) best = best_s[w];
        tokens[b] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
    }
}

}  // namespace bo

// launchers used by the batched step (batched_step.cu); declared in batched_ops.cuh
cudaError_t launch_embed(const bf16 *embed, const int *tokens, bf16 *hidden, int batch, int hidden_size, cudaStream_t st) {
    bo::embed_kernel<<<batch, 128, 0, st>>>(embed, tokens, hidden, hidden_size);
    return cudaGetLastError();
}

cudaError_t launch_residual_norm(bf16 *hidden, const bo::LinOut &lin, int add, const bf16 *weight, bf16 *normed, int batch,
                                 int hidden_size, float eps, cudaStream_t st) {
    bo::residual_norm_kernel<<<batch, bo::kNormThreads, hidden_size * sizeof(float), st>>>(hidden, lin, add, weight, normed,
                                                                                             hidden_size, eps);
    return cudaGetLastError();
}

cudaError_t launch_rope_append(const bo::LinOut &qkv, const int *pos_ids, const float *rope_cos, const float *rope_sin, bf16 *q_out,
                               bf16 *k_cache, bf16 *v_cache, int layer, int rows, int cache_batch, int kv_len, int hq, int hkv,
                               int hd, int half_split, int slot_fixed, cudaStream_t st) {
    bo::rope_append_kernel<<<rows, 256, 0, st>>>(qkv, pos_ids, rope_cos, rope_sin, q_out, k_cache, v_cache, layer, cache_batch,
                                                  kv_len, hq, hkv, hd, half_split, slot_fixed);
    return cudaGetLastError();
}

namespace bo {

// dst[i] = value + i * step
__global__ void fill_int_kernel(int *__restrict__ dst, int value, int step, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value + i * step;
}

// Final values of the batched instruction set's dependency counters
// (megakernels/demos/throughput/python_vm.py: each solver's closing update) for
// the operators a schedule covers.  barriers [layers, 10, batch, cols]; row
// index = 128-sequence block.  One CTA per (layer, opcode - 1); covered[layer]
// has bit (opcode - 1) set for covered operators.
__global__ void barrier_fill_kernel(int *__restrict__ barriers, const int *__restrict__ covered, int batch, int cols,
                                    int batch_blocks, int hq, int hkv, int out_blocks, int inter_blocks) {
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

cudaError_t launch_fill_int(int *dst, int value, int step, int n, cudaStream_t st) {
    bo::fill_int_kernel<<<(n + 255) / 256, 256, 0, st>>>(dst, value, step, n);
    return cudaGetLastError();
}

cudaError_t launch_barrier_fill(int *barriers, const int *covered, int layers, int batch, int cols, int batch_blocks, int hq,
                                int hkv, int out_blocks, int inter_blocks, cudaStream_t st) {
    bo::barrier_fill_kernel<<<layers * 10, 128, 0, st>>>(barriers, covered, batch, cols, batch_blocks, hq, hkv, out_blocks,
                                                        inter_blocks);
    return cudaGetLastError();
}

// Cache splits per (sequence, KV head): enough CTAs to fill the GPU a few times over at small
// batch, none at large batch; at most `max_splits` (what the caller's partial buffer holds).
int attention_batched_splits(int batch, int hkv, int sms, int max_splits) {
    int splits = 1;
    while (batch * hkv * splits < 4 * sms && splits * 2 <= max_splits) splits *= 2;
    return splits;
}

cudaError_t launch_attention_batched(const bf16 *q, const bf16 *k_cache, const bf16 *v_cache, const int *pos_ids, bf16 *out,
                                     float *partial, int splits, int layer, int batch, int cache_batch, int kv_len, int hq, int hkv,
                                     int hd, float attn_scale, int slot_fixed, cudaStream_t st) {
    const dim3 grid(hkv, batch, splits), block(bo::kAttnWarps * 32);
    if (hd == 64)
        bo::attention_batched_kernel<8><<<grid, block, 0, st>>>(q, k_cache, v_cache, pos_ids, out, partial, splits, layer,
                                                                 cache_batch, kv_len, hq, hkv, attn_scale, slot_fixed);
    else
        bo::attention_batched_kernel<16><<<grid, block, 0, st>>>(q, k_cache, v_cache, pos_ids, out, partial, splits, layer,
                                                                  cache_batch, kv_len, hq, hkv, attn_scale, slot_fixed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || splits == 1) return e;
    bo::attention_merge_kernel<<<dim3(hq, batch), hd, 0, st>>>(partial, out, splits, hq, hd);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const bo::LinOut &up, const bo::LinOut &gate, bf16 *act, int batch, int inter, int round_silu,
                            cudaStream_t st) {
    const size_t total = (size_t)batch * inter;
    const size_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    bo::silu_mul_kernel<<<blocks, 256, 0, st>>>(up, gate, act, batch, inter, round_silu);
    return cudaGetLastError();
}

cudaError_t launch_argmax(const bf16 *logits, int *tokens, int batch, int vocab, cudaStream_t st) {
    bo::argmax_kernel<<<batch, 256, 0, st>>>(logits, tokens, vocab);
    return cudaGetLastError();
}

}  // namespace mk
