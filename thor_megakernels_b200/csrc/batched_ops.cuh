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

cudaError_t launch_embed(const bf16 *embed, const int *tokens, bf16 *hidden, int batch, int hidden_size, cudaStream_t st);
cudaError_t launch_residual_norm(bf16 *hidden, const bo::LinOut &lin, int add, const bf16 *weight, bf16 *normed, int batch,
                                 int hidden_size, float eps, cudaStream_t st);
cudaError_t launch_rope_append(const bo::LinOut &qkv, const int *pos_ids, const float *rope_cos, const float *rope_sin, bf16 *q_out,
                               bf16 *k_cache, bf16 *v_cache, int layer, int batch, int kv_len, int hq, int hkv, int hd,
                               cudaStream_t st);
cudaError_t launch_attention_batched(const bf16 *q, const bf16 *k_cache, const bf16 *v_cache, const int *pos_ids, bf16 *out,
                                     int layer, int batch, int kv_len, int hq, int hkv, int hd, float attn_scale,
                                     cudaStream_t st);
cudaError_t launch_silu_mul(const bo::LinOut &up, const bo::LinOut &gate, bf16 *act, int batch, int inter, int round_silu,
                            cudaStream_t st);
cudaError_t launch_argmax(const bf16 *logits, int *tokens, int batch, int vocab, cudaStream_t st);

}  // namespace mk
