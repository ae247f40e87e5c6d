// A prepared chain of NVFP4 x NVFP4 linears: the B200 counterpart of the reference's
// native-FP4 micro-VM surface, experimental/native_fp4_vm/vm.cu:14-63
// (vm_prepare / vm_run / vm_destroy): `length` operands, each a weight matrix in
// NVFP4 (codes + native-layout block scales) applied to a bf16 input panel that
// is either quantised on the fly (the reference's Quantize instruction,
// include/ops/nvfp4_linear.cuh:174-237) or given as NVFP4 already.
//
// The reference schedules Quantize / Linear instructions over at most 20 workers
// of a persistent kernel and orders dependent operands with ready / done
// counters.  Here every operand is one quantiser launch plus one tcgen05
// block-scaled linear that fills the whole GPU, stream order gives the
// dependency, and split-K partials are folded by a small kernel; prepare owns
// all scratch, run allocates nothing.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <new>
#include <vector>

#include "../../include/b200_megakernel.h"
#include "batched_ops.cuh"

extern "C" int32_t mk_linear_batched_splits(int32_t n, int32_t k, int32_t sm_count);

namespace mk {

void set_last_error(const char *msg);  // megakernel.cu

namespace {

struct ChainOp {
    MkFp4ChainOperand o;
    uint8_t *x_packed = nullptr, *x_scales = nullptr;  // quantised input panel (owned when quantising)
    float *partials = nullptr;                        // split-K partial sums (owned)
    int splits = 1;
};

struct Chain {
    std::vector<ChainOp> ops;
    void *scratch = nullptr;
    int *error_word = nullptr;
    int batch = 1;
    bool quantize = false;
};

int fail_chain(int code, const char *text) {
    set_last_error(text);
    return code;
}

// y[b, i] = bf16(sum_s partials[s, b, i])
__global__ void fold_partials_kernel(const float *__restrict__ partials, __nv_bfloat16 *__restrict__ y, int splits, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += partials[(size_t)s * total + idx];
        y[idx] = __float2bfloat16_rn(v);
    }
}

size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace
}  // namespace mk

using namespace mk;

extern "C" int mk_fp4_chain_prepare(const MkFp4ChainOperand *operands, int32_t length, int32_t batch, int32_t quantize,
                                    void **handle) {
    if (!operands || !handle) return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_prepare: null argument");
    *handle = nullptr;
    if (length <= 0 || batch < 1 || batch > 128) return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_prepare: length must be positive and batch 1..128");
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return fail_chain((int)e, cudaGetErrorString(e));
    Chain *c = new (std::nothrow) Chain();
    if (!c) return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_prepare: out of host memory");
    c->batch = batch;
    c->quantize = quantize != 0;
    size_t total = 256;  // error word
    for (int i = 0; i < length; ++i) {
        const MkFp4ChainOperand &o = operands[i];
        // the reference's operand checks (vm.cu:24-27): aligned dimensions, finite positive scales
        if (o.m <= 0 || o.m % 8 || o.k <= 0 || o.k % 256 || !isfinite(o.input_tensor_scale) || !(o.input_tensor_scale > 0.f) ||
            !isfinite(o.alpha)) {
            delete c;
            return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_prepare: operand needs m % 8 == 0, k % 256 == 0, a finite positive input scale and a finite alpha");
        }
        if (!o.output || !o.w_packed || !o.w_scales_native || (c->quantize ? !o.input : (!o.x_packed || !o.x_scales_native))) {
            delete c;
            return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_prepare: operand with a null pointer");
        }
        ChainOp op;
        op.o = o;
        op.splits = mk_linear_batched_splits(o.m, o.k, sms);
        while (op.splits > 1 && ((o.k / 256) % op.splits != 0 || (o.k / 256) / op.splits < 2)) op.splits /= 2;
        if (c->quantize) total += up256((size_t)batch * o.k / 2) + up256((size_t)mk_nvfp4_native_scale_bytes(batch, o.k));
        if (op.splits > 1) total += up256((size_t)op.splits * batch * o.m * sizeof(float));
        c->ops.push_back(op);
    }
    e = cudaMalloc(&c->scratch, total);
    if (e == cudaSuccess) e = cudaMemset(c->scratch, 0, total);
    if (e != cudaSuccess) { if (c->scratch) cudaFree(c->scratch); delete c; return fail_chain((int)e, "mk_fp4_chain_prepare: scratch allocation failed"); }
    uint8_t *at = (uint8_t *)c->scratch;
    c->error_word = (int *)at; at += 256;
    for (ChainOp &op : c->ops) {
        if (c->quantize) {
            op.x_packed = at; at += up256((size_t)batch * op.o.k / 2);
            op.x_scales = at; at += up256((size_t)mk_nvfp4_native_scale_bytes(batch, op.o.k));
        } else {
            op.x_packed = (uint8_t *)op.o.x_packed; op.x_scales = (uint8_t *)op.o.x_scales_native;
        }
        if (op.splits > 1) { op.partials = (float *)at; at += up256((size_t)op.splits * batch * op.o.m * sizeof(float)); }
    }
    *handle = c;
    return 0;
}

extern "C" int mk_fp4_chain_run(void *handle, void *stream) {
    Chain *c = (Chain *)handle;
    if (!c) return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_run: null handle");
    cudaStream_t st = (cudaStream_t)stream;
    for (ChainOp &op : c->ops) {
        const MkFp4ChainOperand &o = op.o;
        if (c->quantize) {
            const int code = mk_nvfp4_quantize_native(o.input, op.x_packed, op.x_scales, c->batch, o.k, o.input_tensor_scale, stream);
            if (code != 0) return code;
        }
        // alpha multiplies the accumulator of decoded codes x decoded block scales (vm.cu:21, nvfp4_linear.cuh:147)
        const int code = mk_linear_batched_nvfp4(o.w_packed, o.w_scales_native, o.alpha / o.input_tensor_scale, op.x_packed, op.x_scales,
                                                 o.input_tensor_scale, op.splits == 1 ? o.output : nullptr, op.partials, o.m, o.k,
                                                 c->batch, op.splits, c->error_word, stream);
        if (code != 0) return code;
        if (op.splits > 1) {
            const long long total = (long long)c->batch * o.m;
            const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
            const cudaError_t e = launch_pdl(fold_partials_kernel, dim3(blocks), dim3(256), 0, st, (const float *)op.partials,
                                             (__nv_bfloat16 *)o.output, op.splits, total);
            if (e != cudaSuccess) return fail_chain((int)e, cudaGetErrorString(e));
        }
    }
    return 0;
}

extern "C" int mk_fp4_chain_status(void *handle, void *stream) {
    Chain *c = (Chain *)handle;
    if (!c) return fail_chain(MK_ERR_BAD_ARGUMENT, "mk_fp4_chain_status: null handle");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    int word = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&word, c->error_word, sizeof(word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_chain((int)e, cudaGetErrorString(e));
    if (word != 0) {
        cudaMemset(c->error_word, 0, sizeof(int));
        return fail_chain(MK_ERR_DEVICE_WAIT, "a bounded wait inside an NVFP4 linear ran out");
    }
    return 0;
}

extern "C" void mk_fp4_chain_destroy(void *handle) {
    Chain *c = (Chain *)handle;
    if (!c) return;
    cudaFree(c->scratch);
    delete c;
}
