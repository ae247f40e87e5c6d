/*
 * C ABI of the B200 decode megakernel library (libb200mk.so).
 *
 * Everything a host needs to drive one Llama decode step on an sm_100a GPU:
 * plain pointers and sizes, int return codes (0 = success, otherwise a
 * cudaError_t value or one of the MK_ERR_* codes below), no exceptions and no
 * framework types.  All pointers named "device" are CUDA device pointers owned
 * by the caller; the library borrows them for the lifetime of the handle.
 *
 * Each entry point names the interface of the reference project
 * (yiannisha/thor-megakernels) that it stands in for.
 */
#ifndef B200_MEGAKERNEL_H
#define B200_MEGAKERNEL_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_ABI_VERSION 1

/* error codes beyond cudaError_t (which stay below 10000) */
#define MK_ERR_BAD_ARGUMENT 10001  /* null pointer, negative size, ABI version mismatch */
#define MK_ERR_UNSUPPORTED  10002  /* shape the kernel is not built for              */
#define MK_ERR_RESIDENCY    10003  /* grid cannot be co-resident / smem over budget  */
#define MK_ERR_DEVICE_WAIT  10004  /* a bounded device-side wait ran out; see mk_status */

/* mk_step flags */
#define MK_STEP_EMBED          1u  /* layer-0 input is embed_w[*token_in] instead of hidden_states */
#define MK_STEP_RESET_BARRIERS 2u  /* the kernel zeroes `barriers` when it finishes               */
#define MK_STEP_WRITE_TOKEN    4u  /* greedy token (argmax of logits) is written to *token_out     */
#define MK_STEP_TIMINGS        8u  /* per-instruction clock stamps are written to `timings`        */

/* weight formats */
#define MK_WEIGHTS_BF16  0
#define MK_WEIGHTS_NVFP4 1

/*
 * One NVFP4 weight matrix [rows, k]: E2M1 codes two per byte (element 2j in the
 * low nibble), one E4M3 scale byte per 16 consecutive k, one fp32 tensor scale.
 * Layout of the reference quantiser, tools/analysis/nvfp4/primitive.cu:50-75
 * ("packed" and "canonical" outputs).
 */
typedef struct MkNvfp4Matrix {
    const uint8_t *packed;   /* device, [rows, k/2]  */
    const uint8_t *scales;   /* device, [rows, k/16] */
    float tensor_scale;
} MkNvfp4Matrix;

/*
 * Model and buffer table.  Field meaning and dtypes are those of the
 * reference's kernel globals (demos/low-latency-llama/llama.cuh:82-147) and of
 * the 27 positional arguments of its native call
 * (megakernels/demos/latency/mk.py:15-48); shapes are runtime values here.
 */
typedef struct MkModelDesc {
    int32_t abi_version;           /* MK_ABI_VERSION */
    int32_t weight_format;         /* MK_WEIGHTS_* */

    int32_t hidden_size;
    int32_t num_layers;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t intermediate_size;
    int32_t vocab_size;
    float   attn_scale;
    float   rms_norm_eps;

    /* bf16 weights, layer-major stacks (MK_WEIGHTS_BF16) */
    const void *qkv_w;             /* [L, (Hq+2Hkv)*D, hidden] */
    const void *o_w;               /* [L, hidden, Hq*D]        */
    const void *up_w;              /* [L, inter, hidden]       */
    const void *gate_w;            /* [L, inter, hidden]       */
    const void *down_w;            /* [L, hidden, inter]       */
    const void *lm_head_w;         /* [vocab, hidden]          */
    /* norm weights are bf16 in both formats */
    const void *attn_norm_w;       /* [L, hidden] */
    const void *mlp_norm_w;        /* [L, hidden] */
    const void *lm_head_norm_w;    /* [hidden]    */
    const void *embed_w;           /* [vocab, hidden] bf16, may be NULL (then MK_STEP_EMBED is refused) */

    /* NVFP4 weights (MK_WEIGHTS_NVFP4): arrays of num_layers entries, except lm_head */
    const MkNvfp4Matrix *qkv_q;
    const MkNvfp4Matrix *o_q;
    const MkNvfp4Matrix *up_q;
    const MkNvfp4Matrix *gate_q;
    const MkNvfp4Matrix *down_q;
    const MkNvfp4Matrix *lm_head_q; /* one entry */

    /* KV cache [L, kv_batch, kv_max_len, Hkv, D] bf16 (kv_batch sequences, only index 0 is decoded) */
    void   *k_cache;
    void   *v_cache;
    int32_t kv_batch;
    int32_t kv_max_len;

    /* rotary tables fp32 [rope_positions, D], adjacent-pair ("interleaved") column order */
    const float *rope_cos;
    const float *rope_sin;
    int32_t rope_positions;

    /* activation buffers */
    void  *hidden_states;          /* bf16 [hidden]: step input (unless MK_STEP_EMBED) and step output */
    void  *q_post_rope;            /* bf16 [Hq*D] */
    void  *attn_out;               /* bf16 [Hq*D] */
    float *attn_lse_intermediates; /* fp32 [Hq, max_partials]    */
    float *attn_out_intermediates; /* fp32 [Hq, max_partials, D] */
    int32_t max_partials;
    void  *silu_out;               /* bf16 [inter] */
    void  *logits;                 /* bf16 [vocab] */

    /* dependency counters int32 [L, barrier_rows, barrier_cols]; zero before every step */
    int32_t *barriers;
    int32_t barrier_rows;          /* >= 8 */
    int32_t barrier_cols;          /* >= Hq + 2*Hkv */
    int32_t skip_attn_reduction;   /* 1: attention writes attn_out directly (single slice per KV head) */
} MkModelDesc;

/* Launch facts, the fields of the dict the reference's binding returns
 * (include/checked_binding.cuh:68-95) that have a meaning here. */
typedef struct MkLaunchInfo {
    int32_t cooperative_launch;
    int32_t physical_sms;
    int32_t resident_worker_capacity;
    int32_t active_workers;
    int32_t threads_per_cta;
    int32_t consumer_warps;
    int32_t registers_per_thread;
    int32_t local_bytes_per_thread;
    int32_t static_smem_bytes;
    int32_t dynamic_smem_bytes;
    int32_t stage_count;           /* weight ring depth ("page_count")  */
    int32_t stage_bytes;           /* bytes per ring stage ("page_size") */
    int32_t resident_ctas_per_sm;
    int32_t queue_len;
    int64_t scratch_bytes;         /* device memory the handle allocated itself */
    int32_t down_fold_mode;        /* how the attached schedule's down-projection slices meet: 0 folds spread over
                                    * the SMs, 1 folded by the last slice's SM, 2 every SM folds its own rows */
    int32_t reserved;
} MkLaunchInfo;

/* Status words of the last step, written by the device when a bounded wait
 * gives up.  code 0 = clean. */
typedef struct MkStatus {
    int32_t code;      /* 0 ok, 1 dependency counter wait, 2 weight-ring wait, 3 partial-buffer wait, 4 unknown opcode,
                        * 5 activation data (tagged cells of another SM or GPU) never arrived; detail = which kind */
    int32_t worker;    /* CTA index */
    int32_t opcode;
    int32_t slot;      /* position in that worker's queue */
    int32_t detail;    /* counter value seen / stage index */
    int32_t expected;
} MkStatus;

/* sizeof() of the structs above as this library was compiled (0 MkModelDesc,
 * 1 MkLaunchInfo, 2 MkStatus, 3 MkNvfp4Matrix); lets a foreign-language binding
 * verify its own struct layout.  No counterpart in the reference. */
int mk_abi_sizeof(int32_t which);

/* Thread-local description of the last failure (reference: nv_error(),
 * tools/analysis/nvfp4/primitive.cu:98-99). */
const char *mk_last_error(void);

/*
 * Bind a model once.  Replaces the per-call marshalling of 27 tensors into
 * kernel globals that the reference's binding repeats on every step
 * (include/checked_binding.cuh:17-21).  Checks shapes, shared-memory budget and
 * co-residency before anything is launched (checked_binding.cuh:29-67) and
 * allocates the handle's own scratch (split-K partial sums, status words,
 * argmax cell) with cudaMalloc on the current device.
 */
int mk_create(const MkModelDesc *desc, void **handle);

/*
 * Attach the instruction and timing queues: int32 [workers, queue_len, 32] and
 * int32 [workers, queue_len, 128] device tensors as produced by
 * tensorize_instructions (megakernels/scheduler.py:380-413).  workers must not
 * exceed the device's SM count.  May be called again to swap schedules.
 * The queues are copied to the host once and every operand the device uses as
 * an index (opcode, layer, row blocks, column slice, attention slice numbers,
 * list lengths) is range-checked: MK_ERR_BAD_ARGUMENT names the worker and slot
 * of the first bad instruction.  Attention slice numbers must stay below
 * min(32, max_partials).  The lowest layer that appears in the queues reads its
 * input from hidden_states (or the embedding), so a schedule may cover layers
 * l..L-1 only (the reference's layer_limit cuts from the other end).
 */
int mk_set_schedule(void *handle, const int32_t *instructions, int32_t *timings,
                    int32_t workers, int32_t queue_len);

/*
 * Run one decode step at position pos_id on `stream` (a cudaStream_t).
 * Stands in for mk_llama.mk_llama(...) (demos/low-latency-llama/llama.cu:24-53;
 * call site megakernels/demos/latency/mk.py:15-49).  token_in/token_out are
 * device int32 cells used only with MK_STEP_EMBED / MK_STEP_WRITE_TOKEN.
 * Asynchronous; device-side wait failures surface through mk_status.
 */
int mk_step(void *handle, int32_t pos_id, uint32_t flags,
            const int32_t *token_in, int32_t *token_out, void *stream);

/* The reference binding's dry_run=True result (checked_binding.cuh:95). */
int mk_query(void *handle, MkLaunchInfo *info);

/* Synchronises `stream`, copies the status words back and clears them.
 * Returns MK_ERR_DEVICE_WAIT when code != 0.  (Reference: optional
 * MK_GMEM_TIMEOUT_CYCLES trap, include/gmem_barrier.cuh:38-47 - here the
 * kernel returns normally and reports.) */
int mk_status(void *handle, MkStatus *status, void *stream);

/* Budget of every device-side wait in SM clock cycles (default 4e9). */
/* After mk_status reported MK_ERR_DEVICE_WAIT: which warps were inside a bounded wait when the launch
 * gave up.  records receives up to max_records entries of 6 ints (worker, warp, code, opcode, slot,
 * detail; warp 0 = loader, 1..8 = consumers, 9 = storer; codes as in MkStatus), *count the number of
 * waiting warps (may exceed max_records).  Clears the record.  Synchronous host copy. */
int mk_status_detail(void *handle, int32_t *records, int32_t max_records, int32_t *count);
int mk_set_wait_budget(void *handle, int64_t cycles);

/* Tuning knobs without a counterpart in the reference (its equivalents are
 * compile-time constants, include/config.cuh:7-72). */
#define MK_OPT_WAIT_BUDGET_CYCLES 0  /* same as mk_set_wait_budget */
#define MK_OPT_DOWN_FOLD_LAST     3  /* 1: only the instruction of a row block's last column slice folds the slices into the
                                      * residual stream (chosen automatically for queues whose down-projection
                                      * instructions of a layer are not consecutive); 0: folds spread over all SMs */
#define MK_OPT_DOWN_FOLD_LOCAL    4  /* 1 (default): where every queue holds all column slices of its down-projection
                                      * row blocks as consecutive instructions in slice order, the SM adds them to
                                      * the residual itself (same bf16 sequence as the interpreter, no cells parked
                                      * for another SM); 0: always fold across SMs */
#define MK_OPT_COOPERATIVE_LAUNCH 5  /* 1 (default): cooperative launch, the runtime guarantees that all CTAs are
                                      * co-resident (the reference's launch mode); 0: ordinary launch of the same
                                      * grid - the CTAs are co-resident whenever the device runs nothing else
                                      * (one CTA per SM, grid <= SM count); if they are not, CTAs that wait on
                                      * one not yet scheduled do so within the wait budget */
#define MK_OPT_MAX_INFLIGHT_TILES 2  /* weight tiles (64 KiB bf16 / 18 KiB NVFP4) one loader keeps in flight */
#define MK_OPT_EARLY_POLL_SHIFT   1  /* consumers stop watching a dependency counter and poll the data cells
                                      * themselves once it is within target >> shift of its target; 31 = never */
int mk_set_option(void *handle, int32_t option, int64_t value);

/*
 * Tensor parallelism over the GPUs of one node, one process per GPU.  The
 * reference shards only its PyTorch model (megakernels/llama.py:192-207,
 * 308-310, 665-691: q/k/v/up/gate by rows, o/down by columns, heads and FFN
 * divided by tp_size); here the handle of rank r is created on that shard
 * (num_q_heads, num_kv_heads, intermediate_size, vocab_size are the rank's 1/n
 * shares, lm_head_w its rows, embed_w the full table) and the two all-reduces per
 * layer run inside the kernel: every rank stores its partial sums into every
 * GPU's exchange buffer over NVLink peer memory and adds what it received in
 * rank order (bit-identical on all ranks).  MK_STEP_WRITE_TOKEN merges the
 * ranks' greedy candidates the same way; token ids are global.
 *
 *   mk_tp_init    allocates this GPU's exchange buffer and returns its CUDA IPC
 *                 handle (MK_TP_HANDLE_BYTES bytes) for the host to all-gather;
 *   mk_tp_connect takes the world's `count` handles in rank order (count must
 *                 equal the world given to mk_tp_init) and maps the peers.  It
 *                 restarts the launch count, so it also clears the handle's
 *                 hand-off cells: steps made before connecting leave nothing behind.
 *
 * Every rank must then make the same sequence of mk_step calls.
 */
#define MK_TP_HANDLE_BYTES 64
int mk_tp_init(void *handle, int32_t rank, int32_t world, int32_t vocab_offset, void *ipc_handle_out);
int mk_tp_connect(void *handle, const void *ipc_handles, int32_t count);

void mk_destroy(void *handle);

/*
 * NVFP4 quantiser: bf16 [rows, k] -> packed codes, E4M3 block scales and,
 * optionally, the fp32 decode of what was stored.  Same arithmetic and argument
 * order as nv_quantize (tools/analysis/nvfp4/primitive.cu:50-75, :104-111)
 * without the tensor-core-native scale layout.  k must be a multiple of 16.
 */
int mk_nvfp4_quantize(const void *input_bf16, void *packed, void *scales, float *decoded,
                      int32_t rows, int32_t k, float tensor_scale, void *stream);

/*
 * Batch-`batch` GEMV y[b, m] = W[m, k] . x[b, k] with bf16 activations and
 * output, fp32 accumulation.  packed != 0: NVFP4 weight-only (fused
 * dequantise), else bf16 weights in `w`.  Mirrors nv_simt
 * (tools/analysis/nvfp4/primitive.cu:79-96, :112-119) and wo_run
 * (experimental/weight_only_fp4/primitive.cu:78-82); batch is 1..8.
 *
 * The call allocates nothing (the reference's per-call entry points borrow all
 * memory from the caller).  When k > 2048 the K dimension is split over CTAs and
 * the fp32 partial sums go through `workspace`: device memory of at least
 * mk_gemv_workspace_bytes(m, k) bytes, 256-byte aligned, owned by the caller
 * and zeroed by the caller ONCE before its first use (every call leaves it
 * zeroed again).  Calls that may overlap in time (different streams) need
 * different workspaces; calls on one stream can share one.  workspace may be
 * NULL when mk_gemv_workspace_bytes returns 0.  The kernel is launched with
 * programmatic stream serialization: consecutive calls on a stream overlap
 * the end of one with the weight fetch of the next.
 *
 * NVFP4 weights: the activations are converted from bf16 to f16 for the tensor
 * cores (code x block scale is exact in f16).  Values beyond +-65504 are clamped
 * to +-65504 and magnitudes below 2^-24 flush to zero; between 2^-24 and 2^-14
 * they keep fewer than bf16's 8 significant bits.  The decode megakernel's
 * NVFP4 path (MK_WEIGHTS_NVFP4) converts its activations the same way.
 */
int64_t mk_gemv_workspace_bytes(int32_t m, int32_t k);
int mk_gemv(const void *w_bf16, const void *packed, const void *scales, const void *x, void *y,
            int32_t m, int32_t k, float tensor_scale, int32_t is_packed, int32_t batch,
            void *workspace, int64_t workspace_bytes, void *stream);

/*
 * mk_gemv without any allocation (no reference counterpart: the reference has
 * no such call).  Same arguments and results as mk_gemv, but the split-K
 * scratch is a fixed 4 MiB + 16 KiB array inside the library, so the call never
 * reaches cudaMalloc/cudaFree.  Limits: k a multiple of 256; when k > 2048,
 * ceil(m/16) <= 4096 and ceil(k/2048) * 8 * m <= 1048576 (e.g. 8192 x 8192,
 * 16384 x 16384); beyond that MK_ERR_UNSUPPORTED with the sizes in
 * mk_last_error().  The array is shared per device: calls that overlap in time
 * race on it.  The first call on a device resolves the array's address and
 * must happen outside stream capture.
 */
int mk_gemv_static(const void *w_bf16, const void *packed, const void *scales, const void *x, void *y,
                   int32_t m, int32_t k, float tensor_scale, int32_t is_packed, int32_t batch, void *stream);

/*
 * Batched decode linear y[b, n] = sum_k x[b, k] * W[n, k] for 1..128 sequences
 * on the tcgen05 tensor cores: weights are the MMA's A operand in 128-row slabs
 * (TMA tiles with 128-byte swizzle), the activation panel is the B operand
 * (N = batch padded to 16/32/64/128), fp32 accumulators in tensor memory,
 * tcgen05.ld epilogue.  The reference's operator of this shape is the in-VM
 * linear include/ops/nvfp4_linear.cuh:52-173 (TMA operands, tcgen05.mma,
 * TMEM accumulators, :136-160 epilogue); this entry point takes bf16 operands.
 *
 * w [n, k] and x [batch, k] are bf16 row-major device tensors, k a multiple of
 * 64.  splits == 1: y [batch, n] bf16 is written.  splits > 1 (k / 64 must be
 * a multiple of splits): K is divided over `splits` CTAs per slab and fp32
 * partial sums go to partials [splits, batch, n] for the caller's next kernel
 * to add in split order; y is not touched.  mk_linear_batched_splits suggests
 * a split count that gives every SM work.  error_word: a device int32 the
 * caller zeroes; set to 1 if a bounded wait inside the kernel ran out.  The
 * call allocates nothing.
 */
int32_t mk_linear_batched_splits(int32_t n, int32_t k, int32_t sm_count);
int mk_linear_batched(const void *w_bf16, const void *x_bf16, void *y_bf16, float *partials,
                      int32_t n, int32_t k, int32_t batch, int32_t splits, int32_t *error_word, void *stream);

/*
 * The same linear with NVFP4 operands on both sides (tcgen05.mma
 * kind::mxf4nvf4, block scale 16): E2M1 codes two per byte, one UE4M3 scale per
 * 16 consecutive k, applied by the tensor core; y = bf16(acc * w_tensor_scale *
 * x_tensor_scale).  Stands in for the reference's in-VM linear and its
 * activation quantiser, include/ops/nvfp4_linear.cuh:52-173 and :174-237
 * (v = x / tensor_scale, scale = e4m3(max(amax / 6, 2^-9)), code = e2m1(v / scale)).
 *
 * mk_nvfp4_quantize_native quantises a bf16 matrix [rows, k] (k a multiple of
 * 64) into packed [rows, k/2] and block scales in the layout the tensor core
 * reads ("native": 512-byte atoms of 128 rows x 4 k-groups, byte
 * (r % 32) * 16 + (r % 128 / 32) * 4 + g % 4 inside atom (r / 128, g / 4);
 * reference tools/analysis/nvfp4/mixed_format.py:9).  The scale buffer holds
 * mk_nvfp4_native_scale_bytes(rows, k) bytes; the caller zeroes it once, so
 * that rows beyond `rows` in the last atom hold scale 0.  Use it for weights
 * (once) and for the activation panel (every step).
 * mk_linear_batched_nvfp4: k a multiple of 256 (and of 256 * splits).
 */
int64_t mk_nvfp4_native_scale_bytes(int32_t rows, int32_t k);
int mk_nvfp4_quantize_native(const void *input_bf16, void *packed, void *scales_native, int32_t rows, int32_t k,
                             float tensor_scale, void *stream);
int mk_linear_batched_nvfp4(const void *w_packed, const void *w_scales_native, float w_tensor_scale,
                            const void *x_packed, const void *x_scales_native, float x_tensor_scale,
                            void *y_bf16, float *partials, int32_t n, int32_t k, int32_t batch, int32_t splits,
                            int32_t *error_word, void *stream);

/*
 * Batched decode: one step for 1..128 sequences, each at its own position.
 * The operations are those of the reference's batched instruction set
 * (megakernels/demos/throughput/instructions.py:57-223; interpreter
 * throughput/python_vm.py:44-465), except that every sequence has its own
 * position id (the reference uses one pos_id for the whole batch) and the
 * rotary embedding is the adjacent-pair form of the batch-1 path, so one model
 * container serves both.  Linears run on the tcgen05 tensor cores
 * (mk_linear_batched); what lies between them are small stream-ordered kernels.
 *
 * mk_batched_create: `desc` as for mk_create with embed_w and either bf16
 *   weights or MK_WEIGHTS_NVFP4 tables (packed codes + canonical scales as
 *   mk_nvfp4_quantize writes them; the handle keeps its own copy of the scales
 *   in the tensor core's native layout).  With NVFP4 weights the step is W4A4
 *   as in the reference's native FP4 path (experimental/native_fp4_vm/model.cu:
 *   102-200, include/ops/nvfp4_linear.cuh:174-237): before every linear its
 *   bf16 input panel is quantised to NVFP4 (tensor scale set by
 *   mk_batched_set_activation_scale, default 1) and the linear runs as
 *   tcgen05 block-scaled MMA; the SiLU product is rounded once.
 *   k_cache / v_cache [L, kv_batch, kv_max_len, Hkv, D] (mk_step_batched needs kv_batch >= batch);
 *   hidden_states [max_batch, hidden] and logits [max_batch, vocab] (bf16) are
 *   the step's residual-stream and logits outputs.  The other activation
 *   pointers, barriers and counters of `desc` are not used.  Allocates the
 *   handle's workspace with one cudaMalloc.
 * mk_step_batched: tokens_in / pos_ids / tokens_out are device int32 [batch];
 *   sequence b reads cache rows 0..pos_ids[b]-1 of cache slot b, appends its new
 *   row at pos_ids[b] and writes its greedy token (lowest index on ties).
 *   tokens_out may be NULL.  Asynchronous on `stream`; allocates nothing, so it
 *   can be captured in a CUDA graph.  Token ids and positions are clamped on
 *   the device into [0, vocab) and [0, min(kv_max_len, rope_positions)) before
 *   anything indexes with them.
 * mk_batched_status: synchronises `stream`; MK_ERR_DEVICE_WAIT if a bounded
 *   wait inside a linear ran out, MK_ERR_BAD_ARGUMENT if a token id or position
 *   had to be clamped since the last call.
 */
int mk_batched_create(const MkModelDesc *desc, int32_t max_batch, void **handle);
int mk_step_batched(void *handle, const int32_t *tokens_in, const int32_t *pos_ids, int32_t batch,
                    int32_t *tokens_out, void *stream);
int mk_batched_status(void *handle, void *stream);
/*
 * Prompt processing (prefill) on the device, replacing the PyTorch forward of
 * megakernels/scripts/generate.py:125-132.  tokens: device int32 [count]; the
 * prompt occupies positions start_pos .. start_pos+count-1 of cache slot `slot`
 * (the batch-1 megakernel uses slot 0), processed max_batch tokens per pass with
 * causal attention.  token_out (optional, device int32[1]) receives the greedy
 * token after the last prompt position; its logits are row 0 of `logits`, and
 * hidden_states holds the residual streams of the last pass's tokens.  The cache
 * only needs the one slot.  Asynchronous on `stream`; allocates nothing.
 */
int mk_prefill_batched(void *handle, const int32_t *tokens, int32_t count, int32_t slot, int32_t start_pos,
                       int32_t *token_out, void *stream);
int mk_batched_set_activation_scale(void *handle, float tensor_scale);
/* Process-wide: 1 (default) launches the batched path's kernels (linears, batched operators, prefill, the
 * batched instruction set, NVFP4 chains) with the programmatic-stream-serialization attribute, so that a
 * kernel's start-up - for a linear, its first weight tiles - overlaps the tail of the kernel before it;
 * 0 = plain stream order.  Results do not change. */
int mk_batched_set_overlap(int32_t enabled);
void mk_batched_destroy(void *handle);

/*
 * The reference's batched instruction set (opcodes 1-10,
 * megakernels/demos/throughput/instructions.py:57-223) on a batched handle.
 * Replaces the native call of megakernels/demos/throughput/mk.py:7-49 (whose
 * kernel the reference project does not ship).  Semantics are those of the
 * reference's interpreter (throughput/python_vm.py:44-465): one pos_id for the
 * whole batch, half-split rotary embedding (no weight permutation), the down
 * projection added to the residual stream as one bf16 addend, the residual
 * stream read from and left in hidden_states, no embedding and no argmax.
 *
 * mk_throughput_bind: the caller's activation buffers (bf16, row-major
 *   [batch_size, width]; widths: hidden for the three rms_* buffers, Hq*D for
 *   post_ln_rope_q and attn_out, intermediate for silu_out).  batch_size is a
 *   multiple of 128 and at most the cache's batch; the descriptor's
 *   hidden_states / logits given to mk_batched_create must hold batch_size rows
 *   and the handle must have been created with max_batch 128 (sequences are
 *   processed 128 at a time).  barriers (optional) is the instruction set's
 *   counter tensor int32 [layers, 10, batch_size, barrier_cols]: after a step it
 *   holds the final counts of the operators the schedule covers, as the
 *   reference's interpreter leaves them.
 * mk_throughput_set_schedule: instructions int32 [workers, queue_len, 32]
 *   (device) in the reference's wire format.  Copied to the host once and
 *   checked: every operand in range, and every operator (layer, opcode) either
 *   absent or present with all of its instructions - operators run whole, in
 *   opcode order within a layer, whatever their placement in the queues.
 *   MK_ERR_UNSUPPORTED for a partial operator or opcode 7 without opcode 6.
 * mk_step_throughput: one step at `pos_id` on `stream`; allocates nothing.
 */
typedef struct MkThroughputBuffers {
    void *rms_rope_intermediates, *rms_gate_intermediates, *rms_lm_head_intermediates;
    void *post_ln_rope_q, *attn_out, *silu_out;
    int32_t *barriers;
    int32_t barrier_cols;
    int32_t batch_size;
} MkThroughputBuffers;
int mk_throughput_bind(void *handle, const MkThroughputBuffers *buffers);
int mk_throughput_set_schedule(void *handle, const int32_t *instructions, int32_t workers, int32_t queue_len);
int mk_step_throughput(void *handle, int32_t pos_id, void *stream);

/*
 * A prepared chain of NVFP4 x NVFP4 linears: the counterpart of the reference's
 * native-FP4 micro-VM surface, experimental/native_fp4_vm/vm.cu:14-63
 * (vm_prepare / vm_run / vm_destroy).  Operand i computes
 *     output[b, :m] = bf16(alpha * sum_k decode(W)[.., k] * decode(X)[b, k])
 * where decode() is code x block scale (tensor scales are folded into alpha, as
 * in the reference: alpha = weight tensor scale x input tensor scale).  With
 * `quantize` != 0 the bf16 `input` [batch, k] is quantised on the fly with
 * `input_tensor_scale` (the reference's Quantize instruction,
 * include/ops/nvfp4_linear.cuh:174-237); otherwise x_packed / x_scales_native
 * hold the panel already (mk_nvfp4_quantize_native).  Operands run in order on
 * the stream, so output[i] may be input[i + 1] (the reference's `dependent`
 * mode).  The reference's worker count, no-op padding and quantiser-worker
 * arguments have no counterpart: each operand's launches fill the GPU.
 * m % 8 == 0, k % 256 == 0 (the reference's rule), batch 1..128 (the
 * reference's VM is batch 1).  prepare allocates the scratch, run nothing.
 */
typedef struct MkFp4ChainOperand {
    const void *input;            /* bf16 [batch, k]  (quantize != 0) */
    const void *x_packed;         /* NVFP4 codes [batch, k/2] and ...  (quantize == 0) */
    const void *x_scales_native;  /* ... block scales in the native layout */
    void *output;                 /* bf16 [batch, m] */
    const void *w_packed;         /* [m, k/2] */
    const void *w_scales_native;  /* native layout, mk_nvfp4_native_scale_bytes(m, k) bytes */
    int32_t m, k;
    float input_tensor_scale;
    float alpha;
} MkFp4ChainOperand;
int mk_fp4_chain_prepare(const MkFp4ChainOperand *operands, int32_t length, int32_t batch, int32_t quantize, void **handle);
int mk_fp4_chain_run(void *handle, void *stream);
int mk_fp4_chain_status(void *handle, void *stream);
void mk_fp4_chain_destroy(void *handle);

#ifdef __cplusplus
}
#endif
#endif /* B200_MEGAKERNEL_H */
