// Launchers of the memory-bound operators of a batched decode step
// (batched_ops.cu) and of the tensor-core linear (linear_batched.cu).
#pragma once

#include <cuda_runtime.h>

#include "mk_device.cuh"

namespace mk {
namespace bo {

struct LinOut {
    const bf16 *y;
    const float *partials;
    int splits, batch, n;
    float scale;
    int group;  // residual adds only: consecutive splits that form one bf16-rounded addend (0: all of them)
};

}  // namespace bo

// Launch on `st` with the programmatic-stream-serialization attribute (see pdl_wait in
// mk_device.cuh): the kernel may be scheduled while its predecessor is still running.
// mk_batched_set_overlap(0) turns the attribute off (plain stream order).
bool launch_overlap_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = launch_overlap_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

cudaError_t launch_embed(const bf16 *embed, const int *tokens, bf16 *hidden, int batch, int hidden_size, int vocab, int *error,
                         cudaStream_t st);
cudaError_t launch_residual_norm(bf16 *hidden, const bo::LinOut &lin, int add, const bf16 *weight, bf16 *normed, int batch,
                                 int hidden_size, float eps, cudaStream_t st);
cudaError_t launch_rope_append(const bo::LinOut &qkv, const int *pos_ids, const float *rope_cos, const float *rope_sin, bf16 *q_out,
                               bf16 *k_cache, bf16 *v_cache, int layer, int rows, int cache_batch, int kv_len, int hq, int hkv,
                               int hd, int half_split, int slot_fixed, cudaStream_t st);
cudaError_t launch_sanitize_positions(const int *pos_ids, int *pos_out, int batch, int pos_limit, int *error, cudaStream_t st);
cudaError_t launch_fill_int(int *dst, int value, int step, int n, cudaStream_t st);
cudaError_t launch_barrier_fill(int *barriers, const int *covered, int layers, int batch, int cols, int batch_blocks, int hq,
                                int hkv, int out_blocks, int inter_blocks, cudaStream_t st);
int attention_batched_splits(int batch, int hkv, int sms, int max_splits);
cudaError_t launch_attention_batched(const bf16 *q, const bf16 *k_cache, const bf16 *v_cache, const int *pos_ids, bf16 *out,
                                     float *partial, int splits, int layer, int batch, int cache_batch, int kv_len, int hq, int hkv,
                                     int hd, float attn_scale, int slot_fixed, cudaStream_t st);
cudaError_t launch_silu_mul(const bo::LinOut &up, const bo::LinOut &gate, bf16 *act, int batch, int inter, int round_silu,
                            cudaStream_t st);
cudaError_t launch_argmax(const bf16 *logits, int *tokens, int batch, int vocab, cudaStream_t st);

}  // namespace mk
