// One decode step for a batch of sequences with independent cache lengths.
//
// The batch-1 megakernel streams every weight past one activation vector; with
// 16..128 sequences per step each weight row meets a [K, batch] panel and the
// linears are dense contractions, so the step is laid out the other way round:
// the tensor-core linear (linear_batched.cu) for the seven matrices of a layer
// and the LM head, and small memory-bound kernels (batched_ops.cu) for what
// sits between them.  The sequence of operations is the reference's batched
// instruction set (megakernels/demos/throughput/instructions.py:57-223:
// pre-attention norm, QKV matmul + rotary + append, decode attention, o_proj +
// residual, pre-MLP norm, gate / up matmuls + SiLU, down_proj + residual,
// LM-head norm, LM head), one stream-ordered launch per operation and layer -
// a caller captures mk_step_batched in a CUDA graph to pay the launches once.
//
// Unlike the reference's batched interpreter (one pos_id for the whole batch,
// throughput/python_vm.py:88), every sequence carries its own position.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "../../include/b200_megakernel.h"
#include "batched_ops.cuh"

extern "C" int mk_linear_batched(const void *w_bf16, const void *x_bf16, void *y_bf16, float *partials, int32_t n, int32_t k,
                                 int32_t batch, int32_t splits, int32_t *error_word, void *stream);
extern "C" int32_t mk_linear_batched_splits(int32_t n, int32_t k, int32_t sm_count);
extern "C" int64_t mk_nvfp4_native_scale_bytes(int32_t rows, int32_t k);
extern "C" int mk_nvfp4_quantize_native(const void *input_bf16, void *packed, void *scales_native, int32_t rows, int32_t k,
                                        float tensor_scale, void *stream);
extern "C" int mk_linear_batched_nvfp4(const void *w_packed, const void *w_scales_native, float w_tensor_scale, const void *x_packed,
                                       const void *x_scales_native, float x_tensor_scale, void *y_bf16, float *partials,
                                       int32_t n, int32_t k, int32_t batch, int32_t splits, int32_t *error_word, void *stream);

namespace mk {

void set_last_error(const char *msg);  // megakernel.cu

namespace {

// One NVFP4 weight matrix as the tensor-core linear reads it: the caller's packed codes and
// a copy of its block scales re-laid out into 512-byte atoms (owned by the handle).
struct Fp4Weight {
    const uint8_t *packed = nullptr;
    const uint8_t *scales_native = nullptr;
    float tensor_scale = 1.f;
};

// canonical scales [rows, k/16] -> native atoms (see mk_nvfp4_quantize_native); one thread per scale byte
__global__ void scales_to_native_kernel(const uint8_t *__restrict__ canonical, uint8_t *__restrict__ native, int rows, int groups) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * groups) return;
    const int r = (int)(idx / groups), g = (int)(idx % groups);
    const size_t atom = ((size_t)(r / 128) * (groups / 4) + g / 4) * 512;
    native[atom + (r % 32) * 16 + ((r % 128) / 32) * 4 + (g % 4)] = canonical[idx];
}

struct BatchedHandle {
    MkModelDesc d;
    bool fp4 = false;
    float act_scale = 1.0f;            // tensor scale of the activation quantiser (NVFP4 weights only)
    Fp4Weight *w_qkv = nullptr, *w_o = nullptr, *w_up = nullptr, *w_gate = nullptr, *w_down = nullptr;  // [layers] (host arrays)
    Fp4Weight w_lm;
    void *native_scales = nullptr;     // one cudaMalloc holding every matrix's native-layout scales
    uint8_t *x_packed = nullptr, *x_sf = nullptr;  // quantised activation panel of the linear being run
    int max_batch = 0;
    int device = 0, sms = 0;
    int qkv_rows = 0;
    // split-K factor per linear
    int s_qkv = 1, s_o = 1, s_up = 1, s_down = 1;
    int down_group = 0;  // split-K partials of the down projection per 2048-column slice (0: no slice structure)
    // workspace (one cudaMalloc)
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    bf16 *normed = nullptr, *q = nullptr, *attn = nullptr, *act = nullptr;
    bf16 *qkv_y = nullptr, *up_y = nullptr, *gate_y = nullptr;
    float *part_a = nullptr, *part_b = nullptr;  // split-K partial sums (two buffers: up and gate are alive together)
    float *attn_partial = nullptr;               // attention split states [batch, Hq, kMaxAttnSplits, D + 2]
    int *error_word = nullptr;
    // batched instruction set (mk_throughput_*)
    MkThroughputBuffers tp = {};
    bool tp_bound = false, plan_ready = false;
    int covered[256] = {};        // per layer: bit (opcode - 1) set when the schedule holds that operator
    int *covered_dev = nullptr;   // device copy, for the counter fill
    int *pos_uniform = nullptr;   // [128] positions of the rows of a pass (clamped copies of the caller's, or generated)
};

int fail_msg(int code, const char *text) {
    set_last_error(text);
    return code;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

constexpr int kMaxAttnSplits = 16;

}  // namespace
}  // namespace mk

using namespace mk;

extern "C" int mk_batched_create(const MkModelDesc *d, int32_t max_batch, void **out) {
    if (!d || !out) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: null argument");
    *out = nullptr;
    if (d->abi_version != MK_ABI_VERSION) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: ABI version mismatch");
    const bool fp4 = d->weight_format == MK_WEIGHTS_NVFP4;
    if (!fp4 && d->weight_format != MK_WEIGHTS_BF16)
        return fail_msg(MK_ERR_UNSUPPORTED, "mk_batched_create: unknown weight format");
    if (max_batch < 1 || max_batch > 128 || d->kv_batch < 1)
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: max_batch must be 1..128");
    const int H = d->hidden_size, D = d->head_dim;
    if (H <= 0 || H % 64 || d->intermediate_size % 64 || (D != 64 && D != 128) || d->num_q_heads != 4 * d->num_kv_heads ||
        d->num_q_heads * D % 64)
        return fail_msg(MK_ERR_UNSUPPORTED, "mk_batched_create: hidden and intermediate sizes must be multiples of 64, head_dim 64 or 128, 4 query heads per KV head");
    const void *required[] = {d->attn_norm_w, d->mlp_norm_w, d->lm_head_norm_w, d->embed_w, d->k_cache, d->v_cache, d->rope_cos,
                              d->rope_sin, d->hidden_states, d->logits};
    for (const void *ptr : required)
        if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 15))
            return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: null or misaligned device pointer in descriptor");
    if (fp4) {
        if (H % 256 || d->intermediate_size % 256 || d->num_q_heads * D % 256)
            return fail_msg(MK_ERR_UNSUPPORTED, "mk_batched_create: NVFP4 weights need every K to be a multiple of 256");
        const MkNvfp4Matrix *tables[] = {d->qkv_q, d->o_q, d->up_q, d->gate_q, d->down_q, d->lm_head_q};
        for (int ti = 0; ti < 6; ++ti) {
            if (!tables[ti]) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: NVFP4 model without a quantised weight table");
            for (int i = 0; i < (ti == 5 ? 1 : d->num_layers); ++i)
                if (!tables[ti][i].packed || !tables[ti][i].scales || (reinterpret_cast<uintptr_t>(tables[ti][i].packed) & 15) ||
                    !(tables[ti][i].tensor_scale > 0.f))
                    return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: NVFP4 matrix with a null or misaligned pointer or a non-positive scale");
        }
    } else {
        const void *weights[] = {d->qkv_w, d->o_w, d->up_w, d->gate_w, d->down_w, d->lm_head_w};
        for (const void *ptr : weights)
            if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 15))
                return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: null or misaligned bf16 weight pointer");
    }
    BatchedHandle *h = new (std::nothrow) BatchedHandle();
    if (!h) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: out of host memory");
    h->d = *d;
    h->fp4 = fp4;
    h->max_batch = max_batch;
    cudaError_t e = cudaGetDevice(&h->device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&h->sms, cudaDevAttrMultiProcessorCount, h->device);
    if (e != cudaSuccess) { delete h; return fail_msg((int)e, "mk_batched_create: device query failed"); }
    const int qd = d->num_q_heads * D, inter = d->intermediate_size;
    h->qkv_rows = (d->num_q_heads + 2 * d->num_kv_heads) * D;
    h->s_qkv = mk_linear_batched_splits(h->qkv_rows, H, h->sms);
    h->s_o = mk_linear_batched_splits(H, qd, h->sms);
    h->s_up = mk_linear_batched_splits(inter, H, h->sms);
    h->s_down = mk_linear_batched_splits(H, inter, h->sms);
    if (inter % 2048 == 0) {
        // Split the down projection along the interpreter's 2048-column slices (each cut further
        // into 1, 2 or 4 pieces while SMs would otherwise idle), so that the residual add can round
        // and add slice by slice as the interpreter does.
        const int slices = inter / 2048, slabs = (H + 127) / 128;
        int pieces = 1;
        while (slabs * slices * pieces < h->sms && pieces < 4) pieces *= 2;
        h->s_down = slices * pieces;
        h->down_group = pieces;
    }
    if (fp4) {
        // K blocks are 256 columns wide here: keep a split only if it still divides them, with at least 2 blocks each
        auto fit = [](int splits, int k) {
            while (splits > 1 && ((k / 256) % splits != 0 || (k / 256) / splits < 2)) splits /= 2;
            return splits;
        };
        h->s_qkv = fit(h->s_qkv, H); h->s_o = fit(h->s_o, qd); h->s_up = fit(h->s_up, H);
        h->s_down = fit(mk_linear_batched_splits(H, inter, h->sms), inter);
        h->down_group = 0;  // the quantised model adds the whole down projection at once
    }
    const size_t B = max_batch;
    const size_t part_a = (size_t)std::max(std::max(h->s_qkv * h->qkv_rows, h->s_o * H), std::max(h->s_up * inter, h->s_down * H));
    const size_t part_b = (size_t)h->s_up * inter;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += align256(bytes); return at; };
    const size_t o_normed = take(B * H * 2), o_q = take(B * qd * 2), o_attn = take(B * qd * 2), o_act = take(B * inter * 2);
    const size_t o_qkv = take(B * h->qkv_rows * 2), o_up = take(B * inter * 2), o_gate = take(B * inter * 2);
    const size_t o_pa = take(B * part_a * 4), o_pb = take(B * part_b * 4), o_err = take(256);
    const size_t o_ap = take(B * d->num_q_heads * kMaxAttnSplits * (D + 2) * 4);
    const size_t o_cov = take(256 * sizeof(int)), o_pos = take(128 * sizeof(int));
    const int max_k = std::max(std::max(H, qd), inter);
    const size_t o_xp = take(fp4 ? B * max_k / 2 : 0), o_xs = take(fp4 ? (size_t)mk_nvfp4_native_scale_bytes((int)B, max_k) : 0);
    h->workspace_bytes = off;
    e = cudaMalloc(&h->workspace, off);
    if (e != cudaSuccess) { delete h; return fail_msg((int)e, "mk_batched_create: cudaMalloc(workspace) failed"); }
    e = cudaMemset(h->workspace, 0, off);
    if (e != cudaSuccess) { cudaFree(h->workspace); delete h; return fail_msg((int)e, "mk_batched_create: cudaMemset failed"); }
    uint8_t *w = (uint8_t *)h->workspace;
    h->normed = (bf16 *)(w + o_normed); h->q = (bf16 *)(w + o_q); h->attn = (bf16 *)(w + o_attn); h->act = (bf16 *)(w + o_act);
    h->qkv_y = (bf16 *)(w + o_qkv); h->up_y = (bf16 *)(w + o_up); h->gate_y = (bf16 *)(w + o_gate);
    h->part_a = (float *)(w + o_pa); h->part_b = (float *)(w + o_pb); h->error_word = (int *)(w + o_err);
    h->x_packed = w + o_xp; h->x_sf = w + o_xs;
    h->attn_partial = (float *)(w + o_ap);
    h->covered_dev = (int *)(w + o_cov); h->pos_uniform = (int *)(w + o_pos);
    if (fp4) {
        // native-layout copies of every matrix's block scales
        const int L = d->num_layers;
        struct Spec { const MkNvfp4Matrix *table; Fp4Weight **dst; int rows, k; };
        const Spec specs[] = {{d->qkv_q, &h->w_qkv, h->qkv_rows, H}, {d->o_q, &h->w_o, H, qd}, {d->up_q, &h->w_up, inter, H},
                              {d->gate_q, &h->w_gate, inter, H}, {d->down_q, &h->w_down, H, inter}};
        size_t total = (size_t)mk_nvfp4_native_scale_bytes(d->vocab_size, H);
        for (const Spec &sp : specs) total += (size_t)L * (size_t)mk_nvfp4_native_scale_bytes(sp.rows, sp.k);
        e = cudaMalloc(&h->native_scales, total);
        if (e == cudaSuccess) e = cudaMemset(h->native_scales, 0, total);
        if (e != cudaSuccess) { cudaFree(h->workspace); delete h; return fail_msg((int)e, "mk_batched_create: cudaMalloc(native scales) failed"); }
        uint8_t *at = (uint8_t *)h->native_scales;
        auto convert = [&](const MkNvfp4Matrix &m, int rows, int k, Fp4Weight &dst) {
            const long long n = (long long)rows * (k / 16);
            scales_to_native_kernel<<<(unsigned)((n + 255) / 256), 256>>>(m.scales, at, rows, k / 16);
            dst.packed = m.packed; dst.scales_native = at; dst.tensor_scale = m.tensor_scale;
            at += mk_nvfp4_native_scale_bytes(rows, k);
        };
        for (const Spec &sp : specs) {
            *sp.dst = new (std::nothrow) Fp4Weight[L];
            if (!*sp.dst) { cudaFree(h->native_scales); cudaFree(h->workspace); delete h; return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: out of host memory"); }
            for (int l = 0; l < L; ++l) convert(sp.table[l], sp.rows, sp.k, (*sp.dst)[l]);
        }
        convert(d->lm_head_q[0], d->vocab_size, H, h->w_lm);
        e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { cudaFree(h->native_scales); cudaFree(h->workspace); delete h; return fail_msg((int)e, "mk_batched_create: scale re-layout failed"); }
    }
    *out = h;
    return 0;
}

namespace mk {
namespace {

// Buffers one pass works on: `rows` sequences starting at some cache slot.
struct StepBuffers {
    bf16 *hidden, *logits;
    bf16 *normed_attn, *normed_mlp, *normed_head;  // outputs of the three RMSNorms (may all be the same scratch)
    bf16 *q, *attn, *act;
    bf16 *k_cache, *v_cache;                       // already offset to the first sequence's cache slot
};

// Issues the stream-ordered launches of the operators, one method per opcode of
// the reference's batched instruction set.  A residual add (o_proj, down_proj) is
// kept pending and folded into the norm that follows it when there is one.
struct Runner {
    BatchedHandle *h;
    cudaStream_t st;
    StepBuffers b;
    const int *pos_ids;
    int rows;
    int half_split;   // rotary pairing (see rope_append_kernel)
    int slice_down;   // add the down projection 2048-column slice by slice (latency interpreter) or as one addend
    int slot_fixed = -1;  // >= 0: every row reads and appends to this cache slot (rows = tokens of one prompt)
    bo::LinOut pending;
    bool has_pending = false;
    int code = 0;

    bool ok(int c) {
        if (c != 0 && code == 0) {
            code = c;
            if (c < 10000) set_last_error(cudaGetErrorString((cudaError_t)c));
        }
        return code == 0;
    }
    bo::LinOut result(bf16 *y, float *partials, int n, int splits) const {
        bo::LinOut o;
        o.y = y; o.partials = splits > 1 ? partials : nullptr; o.splits = splits; o.batch = rows; o.n = n; o.scale = 1.0f;
        o.group = 0;
        return o;
    }
    int linear(const bf16 *w, const Fp4Weight *q, const bf16 *x, bf16 *y, float *partials, int n, int k, int splits) {
        if (!h->fp4)
            return mk_linear_batched(w, x, splits == 1 ? y : nullptr, splits == 1 ? nullptr : partials, n, k, rows, splits,
                                     h->error_word, st);
        // NVFP4: quantise the activation panel (codes + native-layout block scales), then the block-scaled linear
        const int c = mk_nvfp4_quantize_native(x, h->x_packed, h->x_sf, rows, k, h->act_scale, st);
        if (c != 0) return c;
        return mk_linear_batched_nvfp4(q->packed, q->scales_native, q->tensor_scale, h->x_packed, h->x_sf, h->act_scale,
                                       splits == 1 ? y : nullptr, splits == 1 ? nullptr : partials, n, k, rows, splits,
                                       h->error_word, st);
    }
    void norm(const bf16 *weight, bf16 *normed) {
        const MkModelDesc &d = h->d;
        bo::LinOut none = result(nullptr, nullptr, d.hidden_size, 1);
        ok(launch_residual_norm(b.hidden, has_pending ? pending : none, has_pending ? 1 : 0, weight, normed, rows, d.hidden_size,
                                d.rms_norm_eps, st));
        has_pending = false;
    }
    void flush() {  // a pending residual add with no norm behind it
        if (has_pending) norm(nullptr, nullptr);
    }
    void attn_norm(int l) {
        if (code == 0) norm((const bf16 *)h->d.attn_norm_w + (size_t)l * h->d.hidden_size, b.normed_attn);
    }
    void qkv(int l) {
        const MkModelDesc &d = h->d;
        flush();
        if (!ok(linear((const bf16 *)d.qkv_w + (size_t)l * h->qkv_rows * d.hidden_size, h->fp4 ? h->w_qkv + l : nullptr,
                       b.normed_attn, h->qkv_y, h->part_a, h->qkv_rows, d.hidden_size, h->s_qkv)))
            return;
        ok(launch_rope_append(result(h->qkv_y, h->part_a, h->qkv_rows, h->s_qkv), pos_ids, d.rope_cos, d.rope_sin, b.q, b.k_cache,
                              b.v_cache, l, rows, d.kv_batch, d.kv_max_len, d.num_q_heads, d.num_kv_heads, d.head_dim, half_split, slot_fixed, st));
    }
    void attention(int l) {
        const MkModelDesc &d = h->d;
        flush();
        if (code) return;
        ok(launch_attention_batched(b.q, b.k_cache, b.v_cache, pos_ids, b.attn, h->attn_partial,
                                    attention_batched_splits(rows, d.num_kv_heads, h->sms, kMaxAttnSplits), l, rows, d.kv_batch,
                                    d.kv_max_len, d.num_q_heads, d.num_kv_heads, d.head_dim, d.attn_scale, slot_fixed, st));
    }
    void o_proj(int l) {
        const MkModelDesc &d = h->d;
        const int H = d.hidden_size, qd = d.num_q_heads * d.head_dim;
        flush();
        if (code) return;
        if (!ok(linear((const bf16 *)d.o_w + (size_t)l * H * qd, h->fp4 ? h->w_o + l : nullptr, b.attn, h->qkv_y, h->part_a, H, qd,
                       h->s_o)))
            return;
        pending = result(h->qkv_y, h->part_a, H, h->s_o);
        has_pending = true;
    }
    void mlp_norm(int l) {
        if (code == 0) norm((const bf16 *)h->d.mlp_norm_w + (size_t)l * h->d.hidden_size, b.normed_mlp);
    }
    void gate_up(int l, bool with_up) {
        const MkModelDesc &d = h->d;
        const int H = d.hidden_size, inter = d.intermediate_size;
        flush();
        if (code) return;
        bo::LinOut up = result(nullptr, nullptr, inter, 1);
        if (with_up) {
            if (!ok(linear((const bf16 *)d.up_w + (size_t)l * inter * H, h->fp4 ? h->w_up + l : nullptr, b.normed_mlp, h->up_y,
                           h->part_a, inter, H, h->s_up)))
                return;
            up = result(h->up_y, h->part_a, inter, h->s_up);
        }
        if (!ok(linear((const bf16 *)d.gate_w + (size_t)l * inter * H, h->fp4 ? h->w_gate + l : nullptr, b.normed_mlp, h->gate_y,
                       h->part_b, inter, H, h->s_up)))
            return;
        // the quantised model rounds the SiLU product once (tools/analysis/nvfp4/model_reference.py:39-61)
        ok(launch_silu_mul(up, result(h->gate_y, h->part_b, inter, h->s_up), b.act, rows, inter, h->fp4 ? 0 : 1, st));
    }
    void down_proj(int l) {
        const MkModelDesc &d = h->d;
        const int H = d.hidden_size, inter = d.intermediate_size;
        flush();
        if (code) return;
        if (!ok(linear((const bf16 *)d.down_w + (size_t)l * H * inter, h->fp4 ? h->w_down + l : nullptr, b.act, h->qkv_y, h->part_a,
                       H, inter, h->s_down)))
            return;
        pending = result(h->qkv_y, h->part_a, H, h->s_down);
        pending.group = slice_down ? h->down_group : 0;
        has_pending = true;
    }
    void head_norm() {
        if (code == 0) norm((const bf16 *)h->d.lm_head_norm_w, b.normed_head);
    }
    void head() {
        const MkModelDesc &d = h->d;
        flush();
        if (code) return;
        ok(linear((const bf16 *)d.lm_head_w, h->fp4 ? &h->w_lm : nullptr, b.normed_head, b.logits, nullptr, d.vocab_size,
                  d.hidden_size, 1));
    }
};

}  // namespace
}  // namespace mk

extern "C" int mk_step_batched(void *handle, const int32_t *tokens_in, const int32_t *pos_ids, int32_t batch,
                               int32_t *tokens_out, void *stream) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !tokens_in || !pos_ids) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_batched: null argument");
    if (batch < 1 || batch > h->max_batch) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_batched: batch outside 1..max_batch");
    const MkModelDesc &d = h->d;
    if (batch > d.kv_batch) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_batched: the cache holds fewer sequences than the batch");
    Runner r;
    // the kernels index with clamped copies of the caller's positions (bit 1 of the error word if any was out of range)
    r.h = h; r.st = (cudaStream_t)stream; r.pos_ids = h->pos_uniform; r.rows = batch; r.half_split = 0; r.slice_down = 1;
    r.b = StepBuffers{(bf16 *)d.hidden_states, (bf16 *)d.logits, h->normed, h->normed, h->normed, h->q, h->attn, h->act,
                      (bf16 *)d.k_cache, (bf16 *)d.v_cache};
    r.ok(launch_sanitize_positions(pos_ids, h->pos_uniform, batch, std::min(d.kv_max_len, d.rope_positions), h->error_word, r.st));
    r.ok(launch_embed((const bf16 *)d.embed_w, tokens_in, r.b.hidden, batch, d.hidden_size, d.vocab_size, h->error_word, r.st));
    for (int l = 0; l < d.num_layers && r.code == 0; ++l) {
        r.attn_norm(l); r.qkv(l); r.attention(l); r.o_proj(l); r.mlp_norm(l); r.gate_up(l, true); r.down_proj(l);
    }
    r.head_norm();
    r.head();
    if (tokens_out && r.code == 0) r.ok(launch_argmax((const bf16 *)d.logits, tokens_out, batch, d.vocab_size, r.st));
    return r.code;
}

// Prompt processing on the device: the prompt's tokens are the rows of batched passes (up to
// max_batch tokens each) that all use one cache slot; row i sits at position start_pos + i, its
// K / V rows are appended before the pass's attention runs, and attention of row i reads rows
// 0..start_pos + i, which makes it causal.  Replaces the PyTorch forward the reference uses for
// prefill (megakernels/scripts/generate.py:125-132, llama.py:192-207).
extern "C" int mk_prefill_batched(void *handle, const int32_t *tokens, int32_t count, int32_t slot, int32_t start_pos,
                                  int32_t *token_out, void *stream) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !tokens) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_prefill_batched: null argument");
    const MkModelDesc &d = h->d;
    if (count < 1 || slot < 0 || slot >= d.kv_batch || start_pos < 0 || start_pos + count > d.kv_max_len ||
        start_pos + count > d.rope_positions)
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_prefill_batched: prompt outside the cache / rotary tables, or slot outside the cache");
    cudaStream_t st = (cudaStream_t)stream;
    for (int c0 = 0; c0 < count; c0 += h->max_batch) {
        const int rows = std::min(h->max_batch, count - c0);
        cudaError_t e = launch_fill_int(h->pos_uniform, start_pos + c0, 1, rows, st);
        if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
        Runner r;
        r.h = h; r.st = st; r.pos_ids = h->pos_uniform; r.rows = rows; r.half_split = 0; r.slice_down = 1; r.slot_fixed = slot;
        r.b = StepBuffers{(bf16 *)d.hidden_states, (bf16 *)d.logits, h->normed, h->normed, h->normed, h->q, h->attn, h->act,
                          (bf16 *)d.k_cache, (bf16 *)d.v_cache};
        r.ok(launch_embed((const bf16 *)d.embed_w, tokens + c0, r.b.hidden, rows, d.hidden_size, d.vocab_size, h->error_word, st));
        for (int l = 0; l < d.num_layers && r.code == 0; ++l) {
            r.attn_norm(l); r.qkv(l); r.attention(l); r.o_proj(l); r.mlp_norm(l); r.gate_up(l, true); r.down_proj(l);
        }
        r.flush();
        if (r.code == 0 && c0 + rows == count && token_out) {
            // logits and greedy token of the prompt's last position only (row 0 of `logits`)
            Runner last = r;
            last.rows = 1;
            last.b.hidden = r.b.hidden + (size_t)(rows - 1) * d.hidden_size;
            last.head_norm();
            last.head();
            if (last.code == 0) last.ok(launch_argmax((const bf16 *)d.logits, token_out, 1, d.vocab_size, st));
            r.code = last.code;
        }
        if (r.code != 0) return r.code;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The reference's batched instruction set (opcodes 1-10, megakernels/demos/throughput/
// instructions.py:57-223) executed at operator granularity: a schedule is accepted when it
// covers each operator of a layer either completely or not at all, and the covered operators
// run as the same stream-ordered launches as mk_step_batched, 128 sequences at a time, on the
// caller's buffers, with one position for the whole batch and the half-split rotary form.
// ---------------------------------------------------------------------------------------------

extern "C" int mk_throughput_bind(void *handle, const MkThroughputBuffers *buffers) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !buffers) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_bind: null argument");
    if (h->max_batch < 128) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_bind: the handle must be created with max_batch 128");
    if (buffers->batch_size < 128 || buffers->batch_size % 128 || buffers->batch_size > h->d.kv_batch)
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_bind: batch_size must be a multiple of 128 that fits the cache");
    const void *ptrs[] = {buffers->rms_rope_intermediates, buffers->rms_gate_intermediates, buffers->rms_lm_head_intermediates,
                          buffers->post_ln_rope_q, buffers->attn_out, buffers->silu_out};
    for (const void *ptr : ptrs)
        if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 15))
            return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_bind: null or misaligned buffer");
    if (buffers->barriers && buffers->barrier_cols < std::max(h->d.num_q_heads + 2 * h->d.num_kv_heads, h->d.intermediate_size / 128))
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_bind: barrier rows too short for the QKV heads / intermediate blocks");
    h->tp = *buffers;
    h->tp_bound = true;
    h->plan_ready = false;
    return 0;
}

extern "C" int mk_throughput_set_schedule(void *handle, const int32_t *instructions, int32_t workers, int32_t queue_len) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !instructions) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_set_schedule: null argument");
    if (!h->tp_bound) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_set_schedule: bind the buffers first (mk_throughput_bind)");
    if (workers < 1 || queue_len < 1) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_throughput_set_schedule: empty instruction tensor");
    const MkModelDesc &d = h->d;
    if (d.hidden_size % 128 || d.intermediate_size % 128 || d.vocab_size % 128 || (d.num_kv_heads * d.head_dim) % 128)
        return fail_msg(MK_ERR_UNSUPPORTED, "mk_throughput_set_schedule: the instruction set needs hidden, intermediate, vocabulary and K/V widths that are multiples of 128");
    const size_t words = (size_t)workers * queue_len * 32;
    std::vector<int32_t> host(words);
    cudaError_t e = cudaMemcpy(host.data(), instructions, words * sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    const int L = d.num_layers, B = h->tp.batch_size, nbb = B / 128;
    const int qkv_blocks = h->qkv_rows / 128, out_blocks = d.hidden_size / 128, inter_blocks = d.intermediate_size / 128;
    const int vocab_blocks = d.vocab_size / 128;
    // instructions each operator consists of, and the range of its last operand
    const long long expect[11] = {0, B, (long long)nbb * qkv_blocks, (long long)B * d.num_kv_heads, (long long)nbb * out_blocks, B,
                                  (long long)nbb * inter_blocks, (long long)nbb * inter_blocks, (long long)nbb * out_blocks, B,
                                  (long long)nbb * vocab_blocks};
    const int last_range[11] = {0, 0, qkv_blocks, d.num_kv_heads, out_blocks, 0, inter_blocks, inter_blocks, out_blocks, 0, vocab_blocks};
    std::vector<long long> seen((size_t)L * 11, 0);
    char msg[200];
    for (int w = 0; w < workers; ++w)
        for (int s = 0; s < queue_len; ++s) {
            const int32_t *ins = host.data() + ((size_t)w * queue_len + s) * 32;
            const int op = ins[0];
            if (op == 0) continue;
            bool good = op >= 1 && op <= 10;
            int layer = 0;
            if (good) {
                // operands: (layer, first sequence | sequence block[, block]) - the LM head has no layer
                const int a = op == 10 ? 0 : ins[1], bidx = op == 10 ? ins[1] : ins[2], c = op == 10 ? ins[2] : ins[3];
                layer = op >= 9 ? L - 1 : a;
                const bool per_sequence = op == 1 || op == 3 || op == 5 || op == 9;
                good = a >= 0 && a < L && bidx >= 0 && bidx < (per_sequence ? B : nbb) &&
                       (last_range[op] == 0 || (c >= 0 && c < last_range[op]));
            }
            if (!good) {
                snprintf(msg, sizeof(msg), "mk_throughput_set_schedule: worker %d slot %d: opcode %d with operands (%d, %d, %d) is outside the model",
                         w, s, op, ins[1], ins[2], ins[3]);
                return fail_msg(MK_ERR_BAD_ARGUMENT, msg);
            }
            seen[(size_t)layer * 11 + op] += 1;
        }
    std::vector<int> covered(L, 0);
    for (int l = 0; l < L; ++l)
        for (int op = 1; op <= 10; ++op) {
            const long long n = seen[(size_t)l * 11 + op];
            if (n == 0) continue;
            if (n != expect[op]) {
                snprintf(msg, sizeof(msg), "mk_throughput_set_schedule: layer %d opcode %d appears %lld times, the whole operator has %lld instructions (operators run whole or not at all)",
                         l, op, n, expect[op]);
                return fail_msg(MK_ERR_UNSUPPORTED, msg);
            }
            covered[l] |= 1 << (op - 1);
        }
    for (int l = 0; l < L; ++l)
        if ((covered[l] & (1 << 6)) && !(covered[l] & (1 << 5))) {
            snprintf(msg, sizeof(msg), "mk_throughput_set_schedule: layer %d has the up matmul (opcode 7) without the gate matmul (opcode 6)", l);
            return fail_msg(MK_ERR_UNSUPPORTED, msg);
        }
    if ((size_t)L > sizeof(h->covered) / sizeof(h->covered[0]))
        return fail_msg(MK_ERR_UNSUPPORTED, "mk_throughput_set_schedule: more than 256 layers");
    memcpy(h->covered, covered.data(), L * sizeof(int));
    e = cudaMemcpy(h->covered_dev, covered.data(), L * sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    h->plan_ready = true;
    return 0;
}

extern "C" int mk_step_throughput(void *handle, int32_t pos_id, void *stream) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_throughput: null handle");
    if (!h->plan_ready) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_throughput: no schedule attached (mk_throughput_set_schedule)");
    const MkModelDesc &d = h->d;
    if (pos_id < 0 || pos_id >= d.kv_max_len || pos_id >= d.rope_positions)
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_throughput: pos_id outside the cache / rotary tables");
    cudaStream_t st = (cudaStream_t)stream;
    const int L = d.num_layers, B = h->tp.batch_size, H = d.hidden_size, qd = d.num_q_heads * d.head_dim;
    cudaError_t e = launch_fill_int(h->pos_uniform, pos_id, 0, 128, st);
    if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    const size_t slot = (size_t)d.kv_max_len * d.num_kv_heads * d.head_dim;  // cache elements per sequence and layer
    for (int bb = 0; bb < B / 128; ++bb) {
        const size_t r0 = (size_t)bb * 128;
        Runner r;
        r.h = h; r.st = st; r.pos_ids = h->pos_uniform; r.rows = 128; r.half_split = 1; r.slice_down = 0;
        r.b = StepBuffers{(bf16 *)d.hidden_states + r0 * H, (bf16 *)d.logits + r0 * d.vocab_size,
                          (bf16 *)h->tp.rms_rope_intermediates + r0 * H, (bf16 *)h->tp.rms_gate_intermediates + r0 * H,
                          (bf16 *)h->tp.rms_lm_head_intermediates + r0 * H, (bf16 *)h->tp.post_ln_rope_q + r0 * qd,
                          (bf16 *)h->tp.attn_out + r0 * qd, (bf16 *)h->tp.silu_out + r0 * d.intermediate_size,
                          (bf16 *)d.k_cache + r0 * slot, (bf16 *)d.v_cache + r0 * slot};
        for (int l = 0; l < L && r.code == 0; ++l) {
            const int c = h->covered[l];
            if (c & 1) r.attn_norm(l);
            if (c & 2) r.qkv(l);
            if (c & 4) r.attention(l);
            if (c & 8) r.o_proj(l);
            if (c & 16) r.mlp_norm(l);
            if (c & 32) r.gate_up(l, (c & 64) != 0);
            if (c & 128) r.down_proj(l);
            if (l == L - 1) {
                if (c & 256) r.head_norm();
                if (c & 512) r.head();
            }
        }
        r.flush();
        if (r.code != 0) return r.code;
    }
    if (h->tp.barriers) {
        e = launch_barrier_fill((int *)h->tp.barriers, h->covered_dev, L, B, h->tp.barrier_cols, B / 128, d.num_q_heads,
                                d.num_kv_heads, H / 128, d.intermediate_size / 128, st);
        if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    }
    return 0;
}

extern "C" int mk_batched_status(void *handle, void *stream) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_status: null handle");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    int word = 0;
    e = cudaMemcpy(&word, h->error_word, sizeof(word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_msg((int)e, cudaGetErrorString(e));
    if (word != 0) {
        cudaMemset(h->error_word, 0, sizeof(int));
        if (word & 1) return fail_msg(MK_ERR_DEVICE_WAIT, "a bounded wait inside a batched linear ran out");
        return fail_msg(MK_ERR_BAD_ARGUMENT, "a token id or position given to a batched step or prefill was outside the vocabulary / the cache and rotary tables; it was clamped");
    }
    return 0;
}

extern "C" int mk_batched_set_activation_scale(void *handle, float tensor_scale) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !(tensor_scale > 0.f)) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_set_activation_scale: null handle or non-positive scale");
    h->act_scale = tensor_scale;
    return 0;
}

extern "C" void mk_batched_destroy(void *handle) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h) return;
    cudaFree(h->workspace);
    if (h->native_scales) cudaFree(h->native_scales);
    delete[] h->w_qkv; delete[] h->w_o; delete[] h->w_up; delete[] h->w_gate; delete[] h->w_down;
    delete h;
}
