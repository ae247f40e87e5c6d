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
    int *error_word = nullptr;
};

int fail_msg(int code, const char *text) {
    set_last_error(text);
    return code;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

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
    if (max_batch < 1 || max_batch > 128 || d->kv_batch < max_batch)
        return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_batched_create: max_batch must be 1..128 and the cache must hold that many sequences");
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

extern "C" int mk_step_batched(void *handle, const int32_t *tokens_in, const int32_t *pos_ids, int32_t batch,
                               int32_t *tokens_out, void *stream) {
    BatchedHandle *h = (BatchedHandle *)handle;
    if (!h || !tokens_in || !pos_ids) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_batched: null argument");
    if (batch < 1 || batch > h->max_batch) return fail_msg(MK_ERR_BAD_ARGUMENT, "mk_step_batched: batch outside 1..max_batch");
    const MkModelDesc &d = h->d;
    cudaStream_t st = (cudaStream_t)stream;
    const int H = d.hidden_size, D = d.head_dim, L = d.num_layers, inter = d.intermediate_size;
    const int qd = d.num_q_heads * D;
    bf16 *hidden = (bf16 *)d.hidden_states;
    const bf16 *qkv_w = (const bf16 *)d.qkv_w, *o_w = (const bf16 *)d.o_w, *up_w = (const bf16 *)d.up_w;
    const bf16 *gate_w = (const bf16 *)d.gate_w, *down_w = (const bf16 *)d.down_w;
    const bf16 *attn_norm = (const bf16 *)d.attn_norm_w, *mlp_norm = (const bf16 *)d.mlp_norm_w;

    // result of linear (n, splits) in the given buffers, as its consumer reads it
    auto result = [&](bf16 *y, float *partials, int n, int splits) {
        bo::LinOut o;
        o.y = y; o.partials = splits > 1 ? partials : nullptr; o.splits = splits; o.batch = batch; o.n = n; o.scale = 1.0f;
        o.group = 0;
        return o;
    };
    auto linear = [&](const bf16 *w, const Fp4Weight *q, const bf16 *x, bf16 *y, float *partials, int n, int k, int splits) {
        if (!h->fp4)
            return mk_linear_batched(w, x, splits == 1 ? y : nullptr, splits == 1 ? nullptr : partials, n, k, batch, splits,
                                     h->error_word, st);
        // NVFP4: quantise the activation panel (codes + native-layout block scales), then the block-scaled linear
        const int code = mk_nvfp4_quantize_native(x, h->x_packed, h->x_sf, batch, k, h->act_scale, st);
        if (code != 0) return code;
        return mk_linear_batched_nvfp4(q->packed, q->scales_native, q->tensor_scale, h->x_packed, h->x_sf, h->act_scale,
                                       splits == 1 ? y : nullptr, splits == 1 ? nullptr : partials, n, k, batch, splits,
                                       h->error_word, st);
    };
    const int round_silu = h->fp4 ? 0 : 1;  // the quantised model rounds the SiLU product once (model_reference.py:39-61)
#define MK_TRY(expr)                                                             \
    do {                                                                         \
        const int code_ = (int)(expr);                                           \
        if (code_ != 0) {                                                        \
            if (code_ < 10000) set_last_error(cudaGetErrorString((cudaError_t)code_)); \
            return code_;                                                        \
        }                                                                        \
    } while (0)

    MK_TRY(launch_embed((const bf16 *)d.embed_w, tokens_in, hidden, batch, H, st));
    bo::LinOut none = result(nullptr, nullptr, H, 1);
    bo::LinOut down_out = none;
    for (int l = 0; l < L; ++l) {
        // pre-attention norm (adds the previous layer's down projection into the residual first)
        MK_TRY(launch_residual_norm(hidden, down_out, l > 0, attn_norm + (size_t)l * H, h->normed, batch, H, d.rms_norm_eps, st));
        MK_TRY(linear(qkv_w + (size_t)l * h->qkv_rows * H, h->fp4 ? h->w_qkv + l : nullptr, h->normed, h->qkv_y, h->part_a,
                      h->qkv_rows, H, h->s_qkv));
        MK_TRY(launch_rope_append(result(h->qkv_y, h->part_a, h->qkv_rows, h->s_qkv), pos_ids, d.rope_cos, d.rope_sin, h->q,
                                  (bf16 *)d.k_cache, (bf16 *)d.v_cache, l, d.kv_batch, d.kv_max_len, d.num_q_heads,
                                  d.num_kv_heads, D, st));
        MK_TRY(launch_attention_batched(h->q, (const bf16 *)d.k_cache, (const bf16 *)d.v_cache, pos_ids, h->attn, l, d.kv_batch,
                                        d.kv_max_len, d.num_q_heads, d.num_kv_heads, D, d.attn_scale, st));
        // o_proj + residual, pre-MLP norm
        MK_TRY(linear(o_w + (size_t)l * H * qd, h->fp4 ? h->w_o + l : nullptr, h->attn, h->qkv_y, h->part_a, H, qd, h->s_o));
        MK_TRY(launch_residual_norm(hidden, result(h->qkv_y, h->part_a, H, h->s_o), 1, mlp_norm + (size_t)l * H, h->normed, batch,
                                    H, d.rms_norm_eps, st));
        // gate / up + SiLU product
        MK_TRY(linear(up_w + (size_t)l * inter * H, h->fp4 ? h->w_up + l : nullptr, h->normed, h->up_y, h->part_a, inter, H, h->s_up));
        MK_TRY(linear(gate_w + (size_t)l * inter * H, h->fp4 ? h->w_gate + l : nullptr, h->normed, h->gate_y, h->part_b, inter, H,
                      h->s_up));
        MK_TRY(launch_silu_mul(result(h->up_y, h->part_a, inter, h->s_up), result(h->gate_y, h->part_b, inter, h->s_up), h->act,
                               batch, inter, round_silu, st));
        // down_proj; its residual add happens in the next norm
        MK_TRY(linear(down_w + (size_t)l * H * inter, h->fp4 ? h->w_down + l : nullptr, h->act, h->qkv_y, h->part_a, H, inter,
                      h->s_down));
        down_out = result(h->qkv_y, h->part_a, H, h->s_down);
        down_out.group = h->down_group;
    }
    MK_TRY(launch_residual_norm(hidden, down_out, 1, (const bf16 *)d.lm_head_norm_w, h->normed, batch, H, d.rms_norm_eps, st));
    MK_TRY(linear((const bf16 *)d.lm_head_w, h->fp4 ? &h->w_lm : nullptr, h->normed, (bf16 *)d.logits, nullptr, d.vocab_size, H, 1));
    if (tokens_out) MK_TRY(launch_argmax((const bf16 *)d.logits, tokens_out, batch, d.vocab_size, st));
#undef MK_TRY
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
        return fail_msg(MK_ERR_DEVICE_WAIT, "a bounded wait inside a batched linear ran out");
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
