// Persistent decode megakernel for Llama-class models on B200 (sm_100a).
//
// One cooperative launch per decode step.  Every CTA (one per SM) walks its own
// queue of 32-word instructions (the tensor tensorize_instructions builds) with
// three warp roles:
//
//   loader   (warp 0, one elected lane)  streams weight tiles into a ring of
//            shared-memory stages with bulk copies.  Weights never depend on
//            activations, so it runs ahead of the math across instruction and
//            dependency boundaries and keeps HBM busy while others wait.
//   consumer (8 warps)  waits for the instruction's dependency counters, loads
//            and normalises the activation vector into registers, and reduces
//            each 16-row x 2048-column tile to per-warp partial sums.
//   storer   (1 warp)   adds the 8 partial sums in fixed order, applies the
//            op's epilogue (RoPE + KV append, residual add, SiLU-gate, logits +
//            argmax), writes global memory and publishes the dependency counter.
//
// Opcodes, word layouts and counter protocol are those of the reference's
// latency instruction set (megakernels/demos/latency/instructions.py:32-196,
// python_vm.py:83-393); arithmetic and bf16 rounding points follow python_vm.py.
// Every device-side wait is bounded: on expiry the CTA records a status word,
// raises a grid-wide abort flag and all waits fall through so that the kernel
// drains and returns.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "../../include/b200_megakernel.h"
#include "mk_device.cuh"
#include "fp4_mma.cuh"

namespace mk {

// ---------------------------------------------------------------------------
// compile-time geometry
// ---------------------------------------------------------------------------
constexpr int kBlockRows = 16;                            // output rows per block
constexpr int kChunkCols = 2048;                          // input columns per tile
constexpr int kRowBytes = kChunkCols * 2;                 // 4 KiB of a weight row per tile
// Rows sit 64 bytes further apart than their length so that the two rows an
// 8-lane shared-memory access phase touches fall into different bank halves.
constexpr int kRowPitch = kRowBytes + 64;
constexpr int kTileBytes = kBlockRows * kRowBytes;        // 64 KiB moved per tile
constexpr int kStageBytes = kBlockRows * kRowPitch;       // shared-memory footprint of a tile
constexpr int kStages = 3;                                // bf16 tiles in flight per SM (192 KiB)
constexpr int kRingBytes = kStages * kStageBytes;
// NVFP4 tile: 16 rows x 1024 code bytes, then 16 rows x 128 scale bytes
constexpr int kFp4CodeRow = kChunkCols / 2;
constexpr int kFp4ScaleRow = kChunkCols / 16;
constexpr int kFp4ScaleOffset = kBlockRows * kFp4CodeRow;
constexpr int kFp4TileBytes = kBlockRows * (kFp4CodeRow + kFp4ScaleRow);  // 18 KiB
constexpr int kFp4Stages = kRingBytes / kFp4TileBytes;                    // 10 tiles in flight
constexpr int kMaxStages = kFp4Stages > kStages ? kFp4Stages : kStages;

template <bool FP4> struct Fmt {
    static constexpr int stages = FP4 ? kFp4Stages : kStages;
    static constexpr int stage_bytes = FP4 ? kFp4TileBytes : kStageBytes;
    static constexpr int tile_tx = FP4 ? kFp4TileBytes : kTileBytes;  // bytes a fill delivers
};
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = (1 + kConsumerWarps + 1) * 32;   // loader + consumers + storer
constexpr int kStorerWarp = 1 + kConsumerWarps;
constexpr int kPartialBufs = 4;
constexpr int kGroup = 4;                                 // query heads per KV head
constexpr int kMaxHeadDim = 128;
constexpr int kInstrWords = 32;
constexpr int kTimingSlots = 128;
constexpr int kConsumerBarrier = 1;                       // named barrier id
constexpr int kSliceCounterRow = 7;                       // barriers[layer, 7, slice]: gate/up blocks done per 2048-column slice
constexpr int kMaxDownSlices = 8;                         // intermediate_size <= 16384
constexpr int kDownGroup = 4;     // row blocks whose slices the merging storer fetches together
constexpr int kFetchPerLane = 6;  // cells per lane in that fetch
constexpr int kMaxRanks = 8;                              // tensor-parallel ranks
constexpr int kTaggedPartials = 32;                       // attention slices per KV head the scratch can hold
constexpr int kLocalBlocks = 8;   // row blocks of one down-projection instruction when its SM folds the slices itself

// timing slots (reference include/util.cuh:225-256)
constexpr int kEvLoaderStart = 5, kEvStorerStart = 9, kEvConsumerStart = 11;
constexpr int kEvAtWait = 44, kEvDoneWait = 45, kEvFirstUse = 49, kEvFirstStore = 50;
constexpr int kEvLastLoad = 51, kEvLastUse = 52, kEvLastStore = 53, kEvOutputReady = 54;

// status codes
constexpr int kFailCounter = 1, kFailRing = 2, kFailPartial = 3, kFailOpcode = 4, kFailData = 5;

struct Params {
    // shapes
    int hidden, layers, hq, hkv, hd, inter, vocab;
    int qkv_rows;
    int kv_batch, kv_len;
    int max_partials;
    int bar_rows, bar_cols;
    int workers, queue_len;
    int pos;
    int skip_attn_reduction;
    unsigned flags;
    float attn_scale, eps;
    long long spin_cycles;
    int max_inflight;  // weight tiles a loader keeps in flight
    int early_shift;  // consumers start polling cells once a counter is within expected >> early_shift of its target (31: never early)
    int o_cols, o_chunks, o_width;  // output projection: input columns (Hq*D), tiles per row block, columns per tile
    int down_width;   // columns of one down-projection slice (multiple of 256, at most 2048)
    int down_slices;  // inter / down_width
    int down_owner_last;  // 1: the last slice's instruction folds a row block at once (see fold_down_blocks)
    int down_local;       // 1: every queue holds all column slices of its row blocks, in slice order: the SM folds them itself
    int down_total;   // (hidden / 16) * down_slices
    int first_layer;  // lowest layer the schedule touches: its input is the step input, not the previous layer's cells
    // weights
    const bf16 *qkv_w, *attn_norm_w, *o_w, *mlp_norm_w, *up_w, *gate_w, *down_w, *lm_norm_w, *lm_w, *embed_w;
    // NVFP4 weights: per-layer tables in device memory (null for bf16 models)
    const MkNvfp4Matrix *q_qkv, *q_o, *q_up, *q_gate, *q_down, *q_lm;
    // 1: every linear output and the SiLU product are rounded once from fp32, the
    // rounding points of the reference's quantised-model oracle
    // (tools/analysis/nvfp4/model_reference.py:39-61); 0: the bf16 interpreter's
    int model_numerics;
    // cache + tables
    bf16 *k_cache, *v_cache;
    const float *rope_cos, *rope_sin;
    // activations
    bf16 *hidden_states, *q_post, *attn_out;
    float *attn_lse, *attn_oi;
    bf16 *silu_out, *logits;
    // queues and counters
    int *bar;
    const int *instructions;
    int *timings;
    // handle-owned scratch
    // Tagged cells (8 bytes: payload + launch tag), one set per layer so that no
    // cell is written twice in a launch.  Two bf16 per cell unless noted.
    unsigned long long *t_resid;    // [L][hidden/2]            residual stream after the attention block
    unsigned long long *t_hidden;   // [L][hidden/2]            residual stream after the MLP block (layer output)
    unsigned long long *t_down;     // [L][down_slices][hidden] one fp32 per cell: down-projection slice sums
    unsigned long long *t_q;        // [L][hq*hd/2]
    unsigned long long *t_k;        // [L][hkv*hd/2]            this token's key row
    unsigned long long *t_v;        // [L][hkv*hd/2]
    unsigned long long *t_attn;     // [L][hq*hd/2]
    unsigned long long *t_silu;     // [L][inter/2]
    unsigned long long *t_oi;       // [L][hq][kTaggedPartials][hd] one fp32 per cell: attention partial outputs
    unsigned long long *t_lse;      // [L][hq][kTaggedPartials]     one fp32 per cell
    // Tensor parallelism: this rank's shapes above are its 1/n share; the partial
    // output-projection and down-projection sums of all ranks meet in exchange
    // buffers, one per GPU, that every rank can write (peer-mapped).
    int tp_rank, tp_world;          // tp_world == 1: no exchange
    int vocab_offset;               // global id of this rank's first vocabulary row
    unsigned long long *xchg[kMaxRanks];  // [rank] -> that GPU's exchange buffer (own entry = local memory)
    unsigned *epoch;                // launch tag, advanced by the last CTA of every launch
    unsigned long long *argmax_key;
    int *done_counter;
    int *status;                    // [0] code [1] worker [2] opcode [3] slot [4] detail [5] expected [7] abort
    int *stuck;                     // [worker][warp][4]: the wait a warp was in when the launch aborted (code, opcode, slot, detail)
    const int *token_in;
    int *token_out;
};

struct __align__(128) Smem {
    uint8_t ring[kRingBytes];
    float attn[kConsumerWarps][kGroup][kMaxHeadDim + 2];
    float partial[kPartialBufs][kConsumerWarps][kBlockRows];
    float red[2][kConsumerWarps];
    __align__(16) bf16 xbuf[2 * kChunkCols];  // normalised activations, re-read in the MMA operand layout
    float down_parts[kDownGroup][kMaxDownSlices][kBlockRows];  // down-projection slices of the blocks being merged
    float down_acc[kLocalBlocks][kBlockRows];                  // running residual / sum of the rows an SM folds by itself
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t pfull[kPartialBufs];
    uint64_t pempty[kPartialBufs];
    int abort_flag;
    int is_last;
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------

__device__ __forceinline__ bool aborted(const Smem &s) { return *reinterpret_cast<const volatile int *>(&s.abort_flag) != 0; }

// Where this warp was waiting when the launch gave up (first record per warp and failure wins).
__device__ __noinline__ void note_stuck(const Params &p, const Smem &s, int code, int opcode, int slot, int detail) {
    if (*reinterpret_cast<const volatile int *>(&s.abort_flag) == 2) return;  // the failure happened in an earlier launch
    int *rec = p.stuck + ((size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * 4;
    if (atomicCAS(rec, 0, code) == 0) {
        rec[1] = opcode;
        rec[2] = slot;
        rec[3] = detail;
    }
}

__device__ __noinline__ void report_failure(const Params &p, Smem &s, int code, int opcode, int slot, int detail,
                                            int expected) {
    note_stuck(p, s, code, opcode, slot, detail);
    if (atomicCAS(&p.status[0], 0, code) == 0) {
        p.status[1] = blockIdx.x;
        p.status[2] = opcode;
        p.status[3] = slot;
        p.status[4] = detail;
        p.status[5] = expected;
    }
    __threadfence();
    atomicExch(&p.status[7], 1);
    *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
}

// Returns when the barrier phase completes, or when the launch is aborting.
__device__ __forceinline__ void wait_mbar(const Params &p, Smem &s, uint64_t *bar, uint32_t parity, int code,
                                          int opcode, int slot, int detail) {
    if (mbar_try_wait(bar, parity)) return;
    if (aborted(s)) return;
    const long long t0 = clock64();
    unsigned it = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++it & 31u) == 0) {
            if (aborted(s)) { note_stuck(p, s, code, opcode, slot, detail); return; }
            if ((it & 1023u) == 0 && ld_relaxed_gpu(&p.status[7]) != 0) {
                *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
                note_stuck(p, s, code, opcode, slot, detail);
                return;
            }
            if (clock64() - t0 > p.spin_cycles) {
                report_failure(p, s, code, opcode, slot, detail, (int)parity);
                return;
            }
        }
    }
}

// One thread polls a dependency counter until it reaches `expected`.  The
// counter is only a hint that the producers' cells are (about to be) valid; the
// data itself is checked cell by cell, so relaxed accesses suffice.
__device__ __forceinline__ void wait_counter(const Params &p, Smem &s, const int *ctr, int expected, int opcode,
                                             int slot) {
    if (aborted(s)) return;
    int v = ld_relaxed_gpu(ctr);
    if (v >= expected) return;
    const long long t0 = clock64();
    unsigned it = 0;
    while (true) {
        __nanosleep(20);
        v = ld_relaxed_gpu(ctr);
        if (v >= expected) return;
        if ((++it & 15u) == 0) {
            if (aborted(s)) { note_stuck(p, s, kFailCounter, opcode, slot, v); return; }
            if (ld_relaxed_gpu(&p.status[7]) != 0) {
                *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
                note_stuck(p, s, kFailCounter, opcode, slot, v);
                return;
            }
            if (clock64() - t0 > p.spin_cycles) {
                report_failure(p, s, kFailCounter, opcode, slot, v, expected);
                return;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// validated loads of tagged cells
// ---------------------------------------------------------------------------

struct Deadline {
    long long t0;
    unsigned it;
};
__device__ __forceinline__ Deadline start_deadline() { return Deadline{clock64(), 0u}; }

// Called between two attempts to read cells that were not all valid.  Returns
// false when the caller must give up (abort raised or budget spent).
__device__ __forceinline__ bool keep_waiting(const Params &p, Smem &s, Deadline &d, int opcode, int slot, int detail) {
    __nanosleep(40);
    if ((++d.it & 7u) == 0) {
        if (aborted(s)) { note_stuck(p, s, kFailData, opcode, slot, detail); return false; }
        if (ld_relaxed_gpu(&p.status[7]) != 0) {
            *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
            note_stuck(p, s, kFailData, opcode, slot, detail);
            return false;
        }
        if (clock64() - d.t0 > p.spin_cycles) {
            report_failure(p, s, kFailData, opcode, slot, detail, 0);
            return false;
        }
    }
    return !aborted(s);
}

// Eight bf16 values = four cells (32 bytes, 32-byte aligned).
__device__ __forceinline__ bool try_load8(const unsigned long long *cells, uint32_t tag, uint4 &out) {
    const ulonglong2 a = ld_tagged2(cells), b = ld_tagged2(cells + 2);
    out = make_uint4(tag_payload(a.x), tag_payload(a.y), tag_payload(b.x), tag_payload(b.y));
    return tag_ok(a.x, tag) & tag_ok(a.y, tag) & tag_ok(b.x, tag) & tag_ok(b.y, tag);
}

// Eight fp32 values = eight cells.
__device__ __forceinline__ bool try_load8f(const unsigned long long *cells, uint32_t tag, float (&out)[8]) {
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const ulonglong2 a = ld_tagged2(cells + 2 * i);
        out[2 * i] = __uint_as_float(tag_payload(a.x));
        out[2 * i + 1] = __uint_as_float(tag_payload(a.y));
        ok &= tag_ok(a.x, tag) & tag_ok(a.y, tag);
    }
    return ok;
}

struct F8 { float v[8]; };

// Slow paths, kept out of line so that their loops do not inflate the register
// footprint of the streaming code around the (almost always successful) first try.
__device__ __noinline__ uint4 load8_slow(const Params &p, Smem &s, const unsigned long long *cells, uint32_t tag,
                                         int opcode, int slot) {
    // Two probes stay in flight, issued about half an L2 round trip apart, and a new one
    // replaces each probe that comes back without the tag: the cells are looked at
    // twice per round trip instead of once, which shortens the time between a
    // producer's store becoming visible and this thread noticing it.
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    Deadline d = start_deadline();
    ulonglong2 a0 = ld_tagged2(cells), a1 = ld_tagged2(cells + 2);
    __nanosleep(250);
    ulonglong2 b0 = ld_tagged2(cells), b1 = ld_tagged2(cells + 2);
    while (true) {
        if (tag_ok(a0.x, tag) & tag_ok(a0.y, tag) & tag_ok(a1.x, tag) & tag_ok(a1.y, tag)) {
            out = make_uint4(tag_payload(a0.x), tag_payload(a0.y), tag_payload(a1.x), tag_payload(a1.y));
            break;
        }
        a0 = b0; a1 = b1;
        b0 = ld_tagged2(cells); b1 = ld_tagged2(cells + 2);
        if ((++d.it & 15u) == 0) {
            if (aborted(s)) { note_stuck(p, s, kFailData, opcode, slot, 8); break; }
            if (ld_relaxed_gpu(&p.status[7]) != 0) {
                *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
                note_stuck(p, s, kFailData, opcode, slot, 8);
                break;
            }
            if (clock64() - d.t0 > p.spin_cycles) {
                report_failure(p, s, kFailData, opcode, slot, 0, 0);
                break;
            }
        }
    }
    return out;
}

__device__ __noinline__ F8 load8f_slow(const Params &p, Smem &s, const unsigned long long *cells, uint32_t tag,
                                       int opcode, int slot) {
    F8 out;
    Deadline d = start_deadline();
    while (keep_waiting(p, s, d, opcode, slot, 1))
        if (try_load8f(cells, tag, out.v)) break;
    return out;
}

__device__ __noinline__ uint32_t load1_slow(const Params &p, Smem &s, const unsigned long long *cell, uint32_t tag,
                                            int opcode, int slot) {
    unsigned long long v = 0;
    Deadline d = start_deadline();
    while (keep_waiting(p, s, d, opcode, slot, 2)) {
        v = ld_tagged1(cell);
        if (tag_ok(v, tag)) break;
    }
    return tag_payload(v);
}

__device__ __forceinline__ void load8_wait(const Params &p, Smem &s, const unsigned long long *cells, uint32_t tag,
                                           uint4 &out, int opcode, int slot) {
    if (try_load8(cells, tag, out) || aborted(s)) return;
    out = load8_slow(p, s, cells, tag, opcode, slot);
}

__device__ __forceinline__ void load8f_wait(const Params &p, Smem &s, const unsigned long long *cells, uint32_t tag,
                                            float (&out)[8], int opcode, int slot) {
    if (try_load8f(cells, tag, out) || aborted(s)) return;
    const F8 r = load8f_slow(p, s, cells, tag, opcode, slot);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = r.v[i];
}

__device__ __forceinline__ uint32_t load1_wait(const Params &p, Smem &s, const unsigned long long *cell, uint32_t tag,
                                               int opcode, int slot) {
    const unsigned long long v = ld_tagged1(cell);
    if (tag_ok(v, tag) || aborted(s)) return tag_payload(v);
    return load1_slow(p, s, cell, tag, opcode, slot);
}

__device__ __forceinline__ int *counter(const Params &p, int layer, int row, int col) {
    return p.bar + ((size_t)layer * p.bar_rows + row) * p.bar_cols + col;
}

// Exchange buffer of a GPU, in 8-byte tagged cells (one fp32 each):
//   [parity 2][which 2][layer][source rank][hidden]   partial sums (which 0: output projection, 1: down projection)
//   [parity 2][source rank][2]                        greedy-token candidates (logit bits, inverted global index)
// Parity = launch tag & 1: a rank can run at most one launch ahead of its peers
// (it needs their partials of the same launch to get through layer 0), so two
// copies keep a fast rank from overwriting cells a slow one still reads.
__device__ __forceinline__ size_t xchg_partial_cells(const Params &p) {
    return (size_t)2 * 2 * p.layers * p.tp_world * p.hidden;
}
__device__ __forceinline__ unsigned long long *xchg_partials(const Params &p, int gpu, uint32_t tag, int which, int layer) {
    return p.xchg[gpu] + ((((size_t)(tag & 1u) * 2 + which) * p.layers + layer) * p.tp_world) * p.hidden;
}
__device__ __forceinline__ unsigned long long *xchg_token(const Params &p, int gpu, uint32_t tag, int source) {
    return p.xchg[gpu] + xchg_partial_cells(p) + ((size_t)(tag & 1u) * p.tp_world + source) * 2;
}

__device__ __forceinline__ const int *instruction_at(const Params &p, int slot) {
    return p.instructions + ((size_t)blockIdx.x * p.queue_len + slot) * kInstrWords;
}

// The 32 words of an instruction, one per lane of a warp.  Every warp fetches the
// NEXT instruction (one 128-byte load) while it still works on the current one
// and reads fields with a shuffle, so that getting to an instruction costs no
// trip to L2 (about a microsecond while weights are streaming).
struct InsWords {
    int w;  // this lane's word
    // word k, the same for all lanes; every lane of the warp must call this together
    __device__ __forceinline__ int operator[](int k) const { return __shfl_sync(0xffffffffu, w, k); }
};

__device__ __forceinline__ InsWords fetch_instruction(const Params &p, int slot, int lane) {
    InsWords iw;
    iw.w = slot < p.queue_len ? __ldg(instruction_at(p, slot) + lane) : 0;
    return iw;
}

// Single-thread variant (the loader): opcode of the instruction in `slot`, 0 beyond the queue.
__device__ __forceinline__ int opcode_at(const Params &p, int slot) {
    return slot < p.queue_len ? __ldg(instruction_at(p, slot)) : 0;
}

__device__ __forceinline__ void stamp(const Params &p, int slot, int event, long long t_start) {
    if (p.flags & MK_STEP_TIMINGS)
        p.timings[((size_t)blockIdx.x * p.queue_len + slot) * kTimingSlots + event] = (int)(clock64() - t_start);
}

// ---------------------------------------------------------------------------
// loader
// ---------------------------------------------------------------------------

template <int STAGES>
struct Ring {
    uint32_t stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
};

// One 16-row x 2048-column weight tile: first byte, row pitch, owning instruction.
// NVFP4: `src` are the codes (two per byte), `scales` the block scales.
struct Tile {
    const uint8_t *src;
    size_t stride_bytes;
    const uint8_t *scales;
    size_t scale_stride;
    int width;  // columns of this tile (multiple of 256, at most 2048)
    int opcode;
    int slot;
};

// Walks a worker's instruction queue and yields its weight tiles in the order
// the consumers use them.
template <int NCH, bool FP4>
struct TileCursor {
    int slot = -1;
    int op = 0;
    // words 0..4 of slot + 1, loaded while the tiles of `slot` are being issued (ahead.x < 0: not loaded yet)
    int4 ahead = make_int4(-1, 0, 0, 0);
    int ahead4 = 0;
    int w1 = 0, w2 = 0, w3 = 0, w4 = 0;  // words 1..4 of the current instruction
    int idx = 0, cnt = 0;   // block position within the instruction
    int sub = 0, nsub = 1;  // tile position within the block
    int first_block = 0;
    const int *ins = nullptr;
    // bf16: element pointers; NVFP4: code / scale byte pointers (second pair = gate matrix of op 5)
    const uint8_t *base = nullptr, *base2 = nullptr, *sbase = nullptr, *sbase2 = nullptr;
    size_t row_elems = 0;   // K of the matrix
    size_t col0 = 0;        // first column (down projection: the instruction's column slice)
    int width = kChunkCols; // columns per tile

    __device__ __forceinline__ void bind(const bf16 *w, const MkNvfp4Matrix *q, size_t layer, size_t layer_elems,
                                         bool second) {
        const uint8_t *b, *sb = nullptr;
        if constexpr (FP4) {
            b = q[layer].packed;
            sb = q[layer].scales;
        } else {
            b = reinterpret_cast<const uint8_t *>(w + layer * layer_elems);
        }
        if (second) { base2 = b; sbase2 = sb; } else { base = b; sbase = sb; }
    }

    __device__ __forceinline__ bool next(const Params &p, Tile &t) {
        while (true) {
            if (idx < cnt) {
                const int block = (op == 5) ? __ldg(ins + 3 + idx) : first_block + idx;
                const bool second = op == 5 && sub >= NCH;
                const size_t col = col0 + (size_t)((op == 6) ? 0 : (op == 4 ? sub : sub % NCH)) * kChunkCols;
                const size_t elem = (size_t)block * kBlockRows * row_elems + col;
                if constexpr (FP4) {
                    t.src = (second ? base2 : base) + elem / 2;
                    t.stride_bytes = row_elems / 2;
                    t.scales = (second ? sbase2 : sbase) + elem / 16;
                    t.scale_stride = row_elems / 16;
                } else {
                    t.src = (second ? base2 : base) + elem * sizeof(bf16);
                    t.stride_bytes = row_elems * sizeof(bf16);
                    t.scales = nullptr;
                    t.scale_stride = 0;
                }
                t.width = width;
                t.opcode = op;
                t.slot = slot;
                if (++sub == nsub) { sub = 0; ++idx; }
                return true;
            }
            if (++slot >= p.queue_len) return false;
            ins = instruction_at(p, slot);
            if (ahead.x < 0) {
                ahead = __ldg(reinterpret_cast<const int4 *>(ins));
                ahead4 = __ldg(ins + 4);
            }
            op = ahead.x; w1 = ahead.y; w2 = ahead.z; w3 = ahead.w; w4 = ahead4;
            if (slot + 1 < p.queue_len) {
                ahead = __ldg(reinterpret_cast<const int4 *>(instruction_at(p, slot + 1)));
                ahead4 = __ldg(instruction_at(p, slot + 1) + 4);
            } else {
                ahead = make_int4(0, 0, 0, 0);
            }
            idx = 0; sub = 0; cnt = 0; nsub = NCH; col0 = 0; width = kChunkCols;
            const size_t hidden = p.hidden;
            switch (op) {
            case 1: {
                const int layer = w1;
                first_block = w2; cnt = w3 - first_block;
                row_elems = hidden;
                bind(p.qkv_w, p.q_qkv, layer, (size_t)p.qkv_rows * hidden, false);
                break;
            }
            case 4: {
                const int layer = w1;
                first_block = w2; cnt = w3 - first_block;
                row_elems = (size_t)p.o_cols;
                nsub = p.o_chunks; width = p.o_width;
                bind(p.o_w, p.q_o, layer, hidden * row_elems, false);
                break;
            }
            case 5: {
                const int layer = w1;
                cnt = w2; nsub = 2 * NCH;  // up tiles, then gate tiles
                row_elems = hidden;
                bind(p.up_w, p.q_up, layer, (size_t)p.inter * hidden, false);
                bind(p.gate_w, p.q_gate, layer, (size_t)p.inter * hidden, true);
                break;
            }
            case 6: {
                const int layer = w1;
                first_block = w2; cnt = w3 - first_block; nsub = 1;
                row_elems = p.inter;
                width = p.down_width;
                col0 = (size_t)w4 * width;
                bind(p.down_w, p.q_down, layer, hidden * row_elems, false);
                break;
            }
            case 7:
                first_block = w1; cnt = w2 - first_block;
                row_elems = hidden;
                bind(p.lm_w, p.q_lm, 0, 0, false);
                break;
            default:
                break;  // attention ops, no-ops and unknown opcodes stream no weights
            }
            if (cnt < 0) cnt = 0;
        }
    }
};

template <int NCH, bool FP4>
__device__ void loader_role(const Params &p, Smem &s, long long t_start) {
    using F = Fmt<FP4>;
    const uint64_t policy = l2_evict_first_policy();
    Ring<F::stages> ring, land;  // next stage to fill / oldest fill not yet known to have landed
    int outstanding = 0;
    uint32_t live = 0;  // stages whose most recent fill was actually issued
    TileCursor<NCH, FP4> tiles;
    Tile t;
    int last_slot = -1;
    while (tiles.next(p, t)) {
        if (t.slot != last_slot) {
            if (last_slot >= 0) stamp(p, last_slot, kEvLastLoad, t_start);
            stamp(p, t.slot, kEvLoaderStart, t_start);
            last_slot = t.slot;
        }
        // Keep at most `max_inflight` tiles outstanding: more than the memory system
        // needs to stay busy only lengthens its queues, and with them the latency of
        // the small loads on the dependency path between SMs.
        // The fills not yet seen to have landed must never span a whole turn of the ring:
        // mbar_try_wait tells phases apart by parity only, so a fill may not be issued
        // into a stage while the previous fill of that same stage is still unobserved
        // (once the new fill lands, the old phase's parity reads "not complete" again).
        const int inflight_limit = p.max_inflight < F::stages ? p.max_inflight : F::stages;
        while (outstanding > 0 && mbar_try_wait(&s.full[land.stage], land.phase)) { land.advance(); --outstanding; }
        while (outstanding >= inflight_limit && !aborted(s)) {
            wait_mbar(p, s, &s.full[land.stage], land.phase, kFailRing, t.opcode, t.slot, (int)land.stage);
            land.advance();
            --outstanding;
        }
        wait_mbar(p, s, &s.empty[ring.stage], ring.phase ^ 1u, kFailRing, t.opcode, t.slot, (int)ring.stage);
        ++outstanding;
        if (aborted(s)) {
            live &= ~(1u << ring.stage);
        } else {
            live |= 1u << ring.stage;
            uint64_t *bar = &s.full[ring.stage];
            const uint32_t code_row = t.width / 2, scale_row = t.width / 16, row_bytes = t.width * 2;
            mbar_arrive_expect_tx(bar, FP4 ? kBlockRows * (code_row + scale_row) : kBlockRows * row_bytes);
            uint8_t *dst = s.ring + ring.stage * F::stage_bytes;
            if constexpr (FP4) {
                // rows of a K=2048 matrix are contiguous: one copy each for codes and scales
                if (t.width == kChunkCols && t.stride_bytes == (size_t)kFp4CodeRow) {
                    bulk_load(dst, t.src, kBlockRows * kFp4CodeRow, bar, policy);
                    bulk_load(dst + kFp4ScaleOffset, t.scales, kBlockRows * kFp4ScaleRow, bar, policy);
                } else {
#pragma unroll 4
                    for (int r = 0; r < kBlockRows; ++r) {
                        bulk_load(dst + r * kFp4CodeRow, t.src + r * t.stride_bytes, code_row, bar, policy);
                        bulk_load(dst + kFp4ScaleOffset + r * kFp4ScaleRow, t.scales + r * t.scale_stride, scale_row,
                                  bar, policy);
                    }
                }
            } else {
#pragma unroll 4
                for (int r = 0; r < kBlockRows; ++r)
                    bulk_load(dst + r * kRowPitch, t.src + r * t.stride_bytes, row_bytes, bar, policy);
            }
        }
        ring.advance();
    }
    if (last_slot >= 0) stamp(p, last_slot, kEvLastLoad, t_start);
    // Never leave the CTA with copies in flight.  In a clean run every fill has
    // been waited for by the consumers; when aborting, wait here (bounded,
    // ignoring the abort flag) for the last fill of every stage.
    if (aborted(s)) {
        for (uint32_t st = 0; st < (uint32_t)F::stages; ++st) {
            if (!(live & (1u << st))) continue;
            const uint32_t ph = st < ring.stage ? ring.phase : (ring.phase ^ 1u);
            const long long t0 = clock64();
            while (!mbar_try_wait(&s.full[st], ph)) {
                if (clock64() - t0 > p.spin_cycles) break;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// consumer
// ---------------------------------------------------------------------------

template <bool FP4>
struct ConsumerState {
    Ring<Fmt<FP4>::stages> ring;
    uint32_t pbuf = 0;
    uint32_t pphase = 0;
    uint32_t norm_toggle = 0;
    __device__ __forceinline__ void advance_partial() {
        if (++pbuf == kPartialBufs) { pbuf = 0; pphase ^= 1u; }
    }
};

// All consumer threads block until `ctr >= expected` (polled by one thread).
__device__ __forceinline__ void consumer_wait(const Params &p, Smem &s, int ctid, const int *ctr, int expected,
                                              int opcode, int slot) {
    // The counter is a hint: once most producers are done, the threads go on to
    // poll the cells they need, which saves the counter's round trip for the last ones.
    const int target = expected - (expected >> p.early_shift);
    if (ctid == 0 && target > 0) wait_counter(p, s, ctr, target, opcode, slot);  // target 0: not even one look at the counter
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
}

// fp32 tensor scale of a quantised matrix (1 for bf16 weights)
__device__ __forceinline__ float matrix_scale(const MkNvfp4Matrix *table, int layer) {
    return table ? __ldg(&table[layer].tensor_scale) : 1.0f;
}
__device__ __forceinline__ float down_scale(const Params &p, int layer) { return matrix_scale(p.q_down, layer); }

// 8 consecutive elements (starting at `idx`, a multiple of 8) of a bf16 vector
// that is either plain memory written before the launch (`plain`: the step input)
// or tagged cells written by other SMs during it.
__device__ __forceinline__ void load_vector8(const Params &p, Smem &s, uint32_t tag, const bf16 *plain,
                                             const unsigned long long *cells, int idx, float (&h)[8], int opcode,
                                             int slot) {
    if (plain != nullptr) {
        ldcg8(plain + idx, h);
        return;
    }
    uint4 raw;
    load8_wait(p, s, cells + idx / 2, tag, raw, opcode, slot);
    unpack8(raw, h);
}

// Activation operand of the tensor-core matvec.  Consumer warp `cw` owns input
// columns [cw*256, +256) of every 2048-column chunk; within the warp, lane
// (g = lane/4, t = lane%4) holds for j = 0..7 the eight bf16 values of columns
// cw*256 + j*32 + t*8 .. +7 (one uint4).  All eight g-groups hold the same
// values: the MMA's eight output columns are copies and only column 0 is kept.
//
// NVFP4 weights use a different assignment because a lane's 32 code bytes of a
// row are contiguous: x[c][j] holds columns cw*256 + t*64 + j*8 .. +7, converted
// to f16 (the MMA's A operand, code x block scale, is exact in f16).
template <bool FP4>
__device__ __forceinline__ int operand_column(int cw, int t, int j) {
    return FP4 ? cw * 256 + t * 64 + j * 8 : cw * 256 + j * 32 + t * 8;
}

template <bool FP4>
__device__ __forceinline__ uint4 operand_convert(uint4 v) {
    if constexpr (FP4) return make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
    else return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    // both inputs already hold bf16-representable values
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
}

// RMSNorm of the residual stream (reference python_vm.py:50-56): fp32
// statistics; the normalised value is rounded to bf16 and then multiplied by the
// bf16 weight with a second rounding.  Thread `ctid` normalises elements
// [c*2048 + ctid*8, +8) of chunk c; the result goes through shared memory to be
// re-read in the operand layout above.
template <int NCH, bool FP4>
__device__ __forceinline__ void load_normed(const Params &p, Smem &s, int ctid, uint32_t &toggle, uint32_t tag,
                                            const bf16 *plain, const unsigned long long *cells, const bf16 *norm_w,
                                            uint4 (&x)[NCH][8], int opcode, int slot) {
    const int lane = ctid & 31, cw = ctid >> 5;
    uint4 wraw[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) wraw[c] = __ldg(reinterpret_cast<const uint4 *>(norm_w + c * kChunkCols + ctid * 8));
    float h[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        load_vector8(p, s, tag, plain, cells, c * kChunkCols + ctid * 8, h[c], opcode, slot);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(h[c][i], h[c][i], ss);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    // Two scratch rows used alternately: a row is rewritten only after the
    // barrier of the following call, which every reader of it has passed.
    float *red = s.red[toggle];
    toggle ^= 1u;
    if (lane == 0) red[cw] = ss;
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) total += red[w];
    const float rstd = 1.0f / sqrtf(total / (float)p.hidden + p.eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        float w[8], y[8];
        unpack8(wraw[c], w);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = round_bf16(w[i] * round_bf16(h[c][i] * rstd));
        const uint4 packed = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                        pack_bf16x2(y[6], y[7]));
        *reinterpret_cast<uint4 *>(&s.xbuf[c * kChunkCols + ctid * 8]) = packed;
    }
    // xbuf is rewritten only after the statistics barrier of the next call,
    // which no thread reaches before it has finished the reads below.
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    const int t = lane & 3;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            x[c][j] = operand_convert<FP4>(lds128(&s.xbuf[c * kChunkCols + operand_column<FP4>(cw, t, j)]));
}

// Operand from tagged cells (two bf16 per cell) of a vector that starts at
// `cells`: attention output for the output projection, one 2048-column slice of
// the SiLU product for the down projection.  Each thread fetches and validates 8
// elements once; the operand layout (in which the 8 row groups of a warp hold the
// same values) is then read from shared memory, so L2 sees every element once per
// SM instead of eight times.  Callers synchronise the consumer warps between the
// previous reads of xbuf and this call (their dependency wait does).
template <int NCH, bool FP4>
__device__ __forceinline__ void load_operand(const Params &p, Smem &s, const unsigned long long *cells, uint32_t tag,
                                             int ctid, int ncols, uint4 (&x)[NCH][8], int opcode, int slot) {
    const int cw = ctid >> 5, t = ctid & 3;
    uint4 mine[NCH];
    uint32_t missing = 0;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        mine[c] = make_uint4(0u, 0u, 0u, 0u);  // columns beyond the vector count as zero
        if (c * kChunkCols + ctid * 8 < ncols && !try_load8(cells + (c * kChunkCols + ctid * 8) / 2, tag, mine[c]))
            missing |= 1u << c;
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        if (missing & (1u << c)) load8_wait(p, s, cells + (c * kChunkCols + ctid * 8) / 2, tag, mine[c], opcode, slot);
        *reinterpret_cast<uint4 *>(&s.xbuf[c * kChunkCols + ctid * 8]) = mine[c];
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            x[c][j] = operand_convert<FP4>(lds128(&s.xbuf[c * kChunkCols + operand_column<FP4>(cw, t, j)]));
}

// One 16-row block: NCH tiles from the ring times the register-resident
// activation operand.  Lane (g, t) feeds rows g and g+8 of the tile straight
// from shared memory as MMA A-fragments: its 16-byte load at column offset
// j*32 + t*8 supplies the k-slots {2t, 2t+1, 2t+8, 2t+9} of two MMAs, and the
// activation operand uses the same column-to-slot assignment, so no shuffle or
// conversion is needed.  The per-warp results (16 rows) go to the storer.
template <int NCH, bool FP4>
__device__ __forceinline__ void consume_block(const Params &p, Smem &s, ConsumerState<FP4> &st, int lane, int cw,
                                              const uint4 (&x)[NCH][8], int opcode, int slot, int nchunks = NCH,
                                              int width = kChunkCols) {
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
    const int g = lane >> 2, t = lane & 3;
    const bool in_tile = cw * 256 < width;  // narrower tiles leave the upper warps without columns
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        if (c >= nchunks) break;
        wait_mbar(p, s, &s.full[st.ring.stage], st.ring.phase, kFailRing, opcode, slot, (int)st.ring.stage);
        const uint8_t *tile = s.ring + st.ring.stage * Fmt<FP4>::stage_bytes;
        if (!in_tile) {
        } else if constexpr (FP4) {
            // 32 code bytes and 4 scale bytes per row: columns cw*256 + t*64 .. +63
            const uint8_t *cg = tile + g * kFp4CodeRow + cw * 128 + t * 32;
            const uint8_t *ch = cg + 8 * kFp4CodeRow;
            const uint8_t *sg = tile + kFp4ScaleOffset + g * kFp4ScaleRow + cw * 16 + t * 4;
            const uint4 codes_g[2] = {lds128(cg), lds128(cg + 16)};
            const uint4 codes_h[2] = {lds128(ch), lds128(ch + 16)};
            const uint32_t sc_g = *reinterpret_cast<const uint32_t *>(sg);
            const uint32_t sc_h = *reinterpret_cast<const uint32_t *>(sg + 8 * kFp4ScaleRow);
            fp4_rows_mma(acc_a, codes_g, codes_h, sc_g, sc_h, x[c]);
        } else {
            const uint8_t *row_g = tile + g * kRowPitch + cw * 512 + t * 16;
            const uint8_t *row_h = row_g + 8 * kRowPitch;
            uint4 wg = lds128(row_g), wh = lds128(row_h);
            uint4 wg1 = lds128(row_g + 64), wh1 = lds128(row_h + 64);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint4 wg2 = wg1, wh2 = wh1;
                if (j + 2 < 8) {  // two column groups of loads stay ahead of the MMAs
                    wg2 = lds128(row_g + (j + 2) * 64);
                    wh2 = lds128(row_h + (j + 2) * 64);
                }
                mma_bf16_16816(acc_a, wg.x, wh.x, wg.y, wh.y, x[c][j].x, x[c][j].y);
                mma_bf16_16816(acc_b, wg.z, wh.z, wg.w, wh.w, x[c][j].z, x[c][j].w);
                wg = wg1; wh = wh1;
                wg1 = wg2; wh1 = wh2;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.empty[st.ring.stage]);
        st.ring.advance();
    }
    wait_mbar(p, s, &s.pempty[st.pbuf], st.pphase ^ 1u, kFailPartial, opcode, slot, (int)st.pbuf);
    if (t == 0) {  // output column 0
        s.partial[st.pbuf][cw][g] = acc_a[0] + acc_b[0];
        s.partial[st.pbuf][cw][g + 8] = acc_a[2] + acc_b[2];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s.pfull[st.pbuf]);
    st.advance_partial();
}

// Decode attention of one KV head's 4 query heads over cache rows
// [t0, t1) (reference python_vm.py:277-346): fp32 scores, softmax and
// weighted sum; bf16 only at the final store.  A warp takes one cache row per
// iteration; lane (h = lane/8, sub = lane%8) owns query head h and DPL head
// dimensions, so a row's dot products need three shuffles and the running
// softmax state of a head lives in one place per warp.
template <int DPL>
__device__ void attention_partial(const Params &p, Smem &s, int ctid, uint32_t tag, const int *ins, int slot,
                                  long long t_start) {
    constexpr int V = DPL / 8;   // 16-byte vectors per row per lane
    constexpr int kDepth = DPL == 8 ? 8 : 4;  // rows per batch per warp (register budget)
    const int lane = ctid & 31, cw = ctid >> 5;
    const int layer = __ldg(ins + 1), kv_head = __ldg(ins + 2), num_partials = __ldg(ins + 3), part = __ldg(ins + 4);
    const int D = p.hd;

    const int seq_len = p.pos + 1;
    const int total_blocks = (seq_len + 15) / 16;
    const int per_partial = (total_blocks + num_partials - 1) / num_partials;
    const int start_block = part * per_partial;
    int end_block = start_block + per_partial;
    if (end_block > total_blocks) end_block = total_blocks;
    const int t0 = start_block * 16;
    int t1 = end_block * 16;
    if (t1 > seq_len) t1 = seq_len;

    const int h = lane >> 3, sub = lane & 7;
    const int d0 = sub * DPL;
    const size_t tok_stride = (size_t)p.hkv * D;
    const size_t layer_off = (size_t)layer * p.kv_batch * p.kv_len * tok_stride + (size_t)kv_head * D + d0;
    const bf16 *kbase = p.k_cache + layer_off;
    const bf16 *vbase = p.v_cache + layer_off;
    const int my_first = t0 + cw;

    // Rows of earlier positions come from the cache (written by earlier launches);
    // this token's row comes from the tagged cells its producers write in this launch.
    const unsigned long long *k_new = p.t_k + ((size_t)layer * p.hkv * D + (size_t)kv_head * D + d0) / 2;
    const unsigned long long *v_new = p.t_v + ((size_t)layer * p.hkv * D + (size_t)kv_head * D + d0) / 2;
    auto load_row = [&](uint4 (&kq)[V], uint4 (&vq)[V], int t) {
        if (t == p.pos) {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                load8_wait(p, s, k_new + 4 * v, tag, kq[v], 2, slot);
                load8_wait(p, s, v_new + 4 * v, tag, vq[v], 2, slot);
            }
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                kq[v] = __ldcg(reinterpret_cast<const uint4 *>(kbase + (size_t)t * tok_stride) + v);
                vq[v] = __ldcg(reinterpret_cast<const uint4 *>(vbase + (size_t)t * tok_stride) + v);
            }
        }
    };

    // Rows below the current position were written by earlier launches: fetch the
    // first kDepth iterations' worth while the Q/K/V producers are still running.
    uint4 kq[kDepth][V], vq[kDepth][V];
#pragma unroll
    for (int j = 0; j < kDepth; ++j) {
        const int t = my_first + j * kConsumerWarps;
#pragma unroll
        for (int v = 0; v < V; ++v) kq[j][v] = vq[j][v] = make_uint4(0u, 0u, 0u, 0u);
        if (t < t1 && t < p.pos) load_row(kq[j], vq[j], t);
    }

    // The rest of a long slice is pulled into L2 now, also before the producers
    // are done: the loop below holds only kDepth rows per warp in registers, too few
    // bytes in flight to cover DRAM latency, but enough to cover an L2 hit.
    {
        const int first = t0 + kDepth * kConsumerWarps, last = min(t1, p.pos);
        const int lines_per_row = D / 64;  // 128-byte lines of one head's K (or V) row
        const bf16 *krow0 = kbase - d0, *vrow0 = vbase - d0;
        const int items = (last - first) * lines_per_row * 2;
        for (int it = ctid; it < items; it += kConsumerThreads) {
            const int row = first + it / (2 * lines_per_row), rem = it % (2 * lines_per_row);
            const bf16 *src = ((rem & 1) ? vrow0 : krow0) + (size_t)row * tok_stride + (rem >> 1) * 64;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
        }
    }

    // No counter wait: Q and the new K/V row arrive in tagged cells, and each
    // thread waits on exactly the cells it reads (one L2 round trip after the
    // producer's store instead of counter poll + load).
    if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);

    uint4 q[V];
    const unsigned long long *q_cells = p.t_q + ((size_t)layer * p.hq * D + (size_t)(kv_head * kGroup + h) * D + d0) / 2;
#pragma unroll
    for (int v = 0; v < V; ++v) load8_wait(p, s, q_cells + 4 * v, tag, q[v], 2, slot);
    if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
    // the row appended by this launch, if it is one of those fetched early
#pragma unroll
    for (int j = 0; j < kDepth; ++j) {
        const int t = my_first + j * kConsumerWarps;
        if (t < t1 && t >= p.pos) load_row(kq[j], vq[j], t);
    }

    float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    const float scale_log2e = p.attn_scale * 1.4426950408889634f;  // softmax in base 2; m is in log2 units
    if (ctid == 0) stamp(p, slot, 55, t_start);  // loop entry (loads issued, not yet consumed)

    // Rows are taken in batches of kDepth per warp.  Within a batch all scores are
    // computed first (independent dot products and shuffles), then one running-max
    // update, then independent exponentials and accumulations: the only serial
    // dependency is one max/rescale per batch instead of one per row.
    const int n_iter = (t1 - t0 + kConsumerWarps - 1) / kConsumerWarps;  // same for every warp
#pragma unroll 1
    for (int base = 0; base < n_iter; base += kDepth) {
        float sc[kDepth];
#pragma unroll
        for (int j = 0; j < kDepth; ++j) {
            float d = 0.f;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                float kf[8];
                unpack8(kq[j][v], kf);
                d = dot8(q[v], kf, d);
            }
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            const int t = my_first + (base + j) * kConsumerWarps;
            sc[j] = (base + j < n_iter && t < t1) ? d * scale_log2e : -INFINITY;
        }
        float mn = m;
#pragma unroll
        for (int j = 0; j < kDepth; ++j) mn = fmaxf(mn, sc[j]);
        if (mn > -INFINITY) {
            const float corr = exp2f(m - mn);  // exp2(-inf) = 0 for the first batch
            l *= corr;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] *= corr;
#pragma unroll
            for (int j = 0; j < kDepth; ++j) {
                const float pr = exp2f(sc[j] - mn);  // 0 for rows outside the slice
                l += pr;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    float vf[8];
                    unpack8(vq[j][v], vf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[8 * v + i] = fmaf(pr, vf[i], acc[8 * v + i]);
                }
            }
            m = mn;
        }
        // next batch (uniform condition: some warp still has rows)
        if (base + kDepth < n_iter) {
#pragma unroll
            for (int j = 0; j < kDepth; ++j) {
                const int t = my_first + (base + kDepth + j) * kConsumerWarps;
                if (t < t1) load_row(kq[j], vq[j], t);
            }
        }
    }
    if (ctid == 0) stamp(p, slot, 56, t_start);  // cache rows consumed

#pragma unroll
    for (int i = 0; i < DPL; ++i) s.attn[cw][h][d0 + i] = acc[i];
    if (sub == 0) {
        s.attn[cw][h][kMaxHeadDim] = m;
        s.attn[cw][h][kMaxHeadDim + 1] = l;
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    if (ctid == 0) stamp(p, slot, 57, t_start);  // per-warp states exchanged

    // merge the 8 warps; one (head, dim) output per thread and iteration.  A warp's 32 outputs belong
    // to one head, so the eight weights exp2(m_w - M) are computed once per warp (lane w holds warp
    // w's state) and handed round by shuffles.
    constexpr int Dc = DPL * 8;
    static_assert(kGroup * Dc % kConsumerThreads == 0 && Dc % 32 == 0, "a warp's outputs must share a head");
#pragma unroll
    for (int it = 0; it < kGroup * Dc / kConsumerThreads; ++it) {
        const int idx = it * kConsumerThreads + ctid;
        const int h = idx / Dc, d = idx % Dc;
        const float mw = lane < kConsumerWarps ? s.attn[lane][h][kMaxHeadDim] : -INFINITY;
        const float lw = lane < kConsumerWarps ? s.attn[lane][h][kMaxHeadDim + 1] : 0.f;
        float M = mw;
#pragma unroll
        for (int off = 4; off; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        M = __shfl_sync(0xffffffffu, M, 0);
        const float fw = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        float L = fw * lw;
#pragma unroll
        for (int off = 4; off; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        L = __shfl_sync(0xffffffffu, L, 0);
        float O = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) O = fmaf(s.attn[w][h][d], __shfl_sync(0xffffffffu, fw, w), O);
        const float out = (L > 0.f) ? O / L : 0.f;
        const int head = kv_head * kGroup + h;
        // neighbouring threads hold neighbouring dimensions: the even one writes the pair's cell
        const float out_bf = round_bf16(out);
        const float next_bf = __shfl_xor_sync(0xffffffffu, out_bf, 1);
        if (!aborted(s)) {
            if (p.skip_attn_reduction) {
                p.attn_out[(size_t)head * D + d] = __float2bfloat16_rn(out);
                if ((d & 1) == 0)
                    st_tagged(p.t_attn + ((size_t)layer * p.hq * D + (size_t)head * D + d) / 2, pack_bf16x2(out_bf, next_bf), tag);
            } else {
                p.attn_oi[((size_t)head * p.max_partials + part) * D + d] = out;
                st_tagged(p.t_oi + (((size_t)layer * p.hq + head) * kTaggedPartials + part) * D + d, __float_as_uint(out), tag);
                // log2 of the natural-exponent sum (reference python_vm.py:323); M is already in log2 units
                if (d == 0) {
                    const float lse = (L > 0.f) ? M + log2f(L) : -INFINITY;
                    p.attn_lse[(size_t)head * p.max_partials + part] = lse;
                    st_tagged(p.t_lse + ((size_t)layer * p.hq + head) * kTaggedPartials + part, __float_as_uint(lse), tag);
                }
            }
        }
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);  // all stores issued; s.attn reusable
    if (ctid == 0) stamp(p, slot, 58, t_start);  // outputs stored
    if (ctid == 0 && !aborted(s)) {
        // hints only: consumers validate the cells themselves
        if (p.skip_attn_reduction) {
            red_relaxed_gpu_add(counter(p, layer, 2, 0), kGroup);
        } else {
            for (int hh = 0; hh < kGroup; ++hh) red_relaxed_gpu_add(counter(p, layer, 1, kv_head * kGroup + hh), 1);
        }
        stamp(p, slot, kEvOutputReady, t_start);
    }
}

// Log-sum-exp merge of attention partials for 4 heads (reference
// python_vm.py:349-393).  Weights are exp2(lse - max); a non-terminal merge
// stores the natural log of the weight sum as the reference does.
__device__ void attention_reduction(const Params &p, Smem &s, int ctid, uint32_t tag, const int *ins, int slot,
                                    long long t_start) {
    const int layer = __ldg(ins + 1), head0 = __ldg(ins + 2), num_partials = __ldg(ins + 3);
    const int terminal = __ldg(ins + 4), n = __ldg(ins + 5);
    const int out_slot = __ldg(ins + 6 + n);
    const int D = p.hd;
    // partials arrive in tagged cells: every thread waits on the cells it reads
    if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
    // The log-sum-exps of the 4 heads' partials go through shared memory (one cell
    // per thread, all in flight together) instead of being re-read by every thread.
    float *lse_s = &s.attn[0][0][0];  // [kGroup][kTaggedPartials]
    if (ctid < kGroup * n) {
        const int h = ctid / n, j = ctid % n;
        const unsigned long long *cell = p.t_lse + ((size_t)layer * p.hq + head0 + h) * kTaggedPartials + __ldg(ins + 6 + j);
        lse_s[h * kTaggedPartials + j] = __uint_as_float(load1_wait(p, s, cell, tag, 3, slot));
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    for (int idx = ctid; idx < kGroup * D; idx += kConsumerThreads) {
        const int h = idx / D, d = idx % D;
        const int head = head0 + h;
        const unsigned long long *oi = p.t_oi + (((size_t)layer * p.hq + head) * kTaggedPartials) * D + d;
        float mx = -INFINITY;
        for (int j = 0; j < n; ++j) mx = fmaxf(mx, lse_s[h * kTaggedPartials + j]);
        float denom = 0.f, num = 0.f;
        // partial outputs: eight independent loads in flight, validated afterwards
        for (int j0 = 0; j0 < n; j0 += 8) {
            unsigned long long raw[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (j0 + u < n) raw[u] = ld_tagged1(oi + (size_t)__ldg(ins + 6 + j0 + u) * D);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j0 + u < n) {
                    uint32_t bits = tag_payload(raw[u]);
                    if (!tag_ok(raw[u], tag)) bits = load1_wait(p, s, oi + (size_t)__ldg(ins + 6 + j0 + u) * D, tag, 3, slot);
                    const float f = exp2f(lse_s[h * kTaggedPartials + j0 + u] - mx);
                    denom += f;
                    num = fmaf(__uint_as_float(bits), f, num);
                }
            }
        }
        const float out = num / denom;
        const float out_bf = round_bf16(out);
        const float next_bf = __shfl_xor_sync(0xffffffffu, out_bf, 1);
        if (!aborted(s)) {
            if (terminal) {
                p.attn_out[(size_t)head * D + d] = __float2bfloat16_rn(out);
                if ((d & 1) == 0)
                    st_tagged(p.t_attn + ((size_t)layer * p.hq * D + (size_t)head * D + d) / 2, pack_bf16x2(out_bf, next_bf), tag);
            } else {
                // intermediate merge level (the schedule builders here only emit terminal merges)
                p.attn_oi[((size_t)head * p.max_partials + out_slot) * D + d] = out;
                st_tagged(p.t_oi + (((size_t)layer * p.hq + head) * kTaggedPartials + out_slot) * D + d, __float_as_uint(out), tag);
                if (d == 0) {
                    p.attn_lse[(size_t)head * p.max_partials + out_slot] = logf(denom);
                    st_tagged(p.t_lse + ((size_t)layer * p.hq + head) * kTaggedPartials + out_slot, __float_as_uint(logf(denom)), tag);
                }
            }
        }
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    if (ctid == 0 && !aborted(s)) {
        red_relaxed_gpu_add(counter(p, layer, 2, 0), kGroup);
        stamp(p, slot, kEvOutputReady, t_start);
    }
}

// The token id is read from device memory, where the host cannot check it: one outside the
// table (whole vocabulary = this rank's rows x ranks) is clamped to its nearest row.
__device__ __forceinline__ const bf16 *embedding_row(const Params &p) {
    const int rows = p.vocab * p.tp_world;
    int t = __ldg(p.token_in);
    t = t < 0 ? 0 : (t >= rows ? rows - 1 : t);
    return p.embed_w + (size_t)t * p.hidden;
}

template <int NCH, bool FP4>
__device__ void consumer_role(const Params &p, Smem &s, int ctid, long long t_start) {
    const int lane = ctid & 31, cw = ctid >> 5;
    ConsumerState<FP4> st;
    const uint32_t tag = __ldg(p.epoch);
    // layer-0 input: the embedding row of the fed-back token, or the host-written hidden state
    const bf16 *step_input = p.hidden_states;
    if (p.flags & MK_STEP_EMBED) step_input = embedding_row(p);

    InsWords next_ins = fetch_instruction(p, 0, lane);
#pragma unroll 1
    for (int slot = 0; slot < p.queue_len; ++slot) {
        const InsWords ins = next_ins;
        next_ins = fetch_instruction(p, slot + 1, lane);  // in flight while this instruction runs
        const int op = ins[0];
        if (op == 0) continue;
        if (ctid == 0) stamp(p, slot, kEvConsumerStart, t_start);
        uint4 x[NCH][8];
        switch (op) {
        case 1: {
            const int layer = ins[1], b0 = ins[2], b1 = ins[3];
            if (layer != p.first_layer) {
                if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
                consumer_wait(p, s, ctid, counter(p, layer - 1, 5, 0), p.down_total, op, slot);
                if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            }
            load_normed<NCH, FP4>(p, s, ctid, st.norm_toggle, tag, layer == p.first_layer ? step_input : nullptr,
                                  p.t_hidden + (size_t)(layer - 1) * (p.hidden / 2),
                                  p.attn_norm_w + (size_t)layer * p.hidden, x, op, slot);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH, FP4>(p, s, st, lane, cw, x, op, slot);
            break;
        }
        case 2:
            if (p.hd == 64) attention_partial<8>(p, s, ctid, tag, instruction_at(p, slot), slot, t_start);
            else attention_partial<16>(p, s, ctid, tag, instruction_at(p, slot), slot, t_start);
            break;
        case 3:
            attention_reduction(p, s, ctid, tag, instruction_at(p, slot), slot, t_start);
            break;
        case 4: {
            const int layer = ins[1], b0 = ins[2], b1 = ins[3];
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, layer, 2, 0), p.hq, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_operand<NCH, FP4>(p, s, p.t_attn + (size_t)layer * (p.o_cols / 2), tag, ctid, p.o_cols, x, op, slot);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH, FP4>(p, s, st, lane, cw, x, op, slot, p.o_chunks, p.o_width);
            break;
        }
        case 5: {
            const int layer = ins[1], n = ins[2];
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, layer, 3, 0), p.hidden / kBlockRows, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_normed<NCH, FP4>(p, s, ctid, st.norm_toggle, tag, nullptr, p.t_resid + (size_t)layer * (p.hidden / 2),
                                  p.mlp_norm_w + (size_t)layer * p.hidden, x, op, slot);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int i = 0; i < n; ++i) {
                consume_block<NCH, FP4>(p, s, st, lane, cw, x, op, slot);  // up rows
                consume_block<NCH, FP4>(p, s, st, lane, cw, x, op, slot);  // gate rows
            }
            break;
        }
        case 6: {
            const int layer = ins[1], b0 = ins[2], b1 = ins[3], red = ins[4];
            if (p.down_local) {
                // This queue holds the instructions of all column slices of rows
                // [b0*16, b1*16) in the next down_slices slots (checked when the schedule
                // was attached).  They are run as one piece: while the tiles of slice r
                // go through the tensor cores, the cells of slice r+1 of the SiLU product
                // are already on their way from L2, so the SM pays the wait for its input
                // once instead of once per slice.  Loader and storer still see one
                // instruction per slice.
                const int S = p.down_slices, width = p.down_width;
                const InsWords after_run = fetch_instruction(p, slot + S, lane);  // what follows the run
                const int t = lane & 3;
                const bool has_cols = ctid * 8 < width;  // narrower slices leave the upper threads without columns
                const unsigned long long *silu = p.t_silu + ((size_t)layer * p.inter) / 2 + (ctid * 8) / 2;
                // One round of loads fetches this thread's 8 values of EVERY slice; slices
                // whose producers are not done yet are fetched again when their turn comes.
                uint4 mine[kMaxDownSlices];
                uint32_t valid = 0;
                if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
#pragma unroll
                for (int r = 0; r < kMaxDownSlices; ++r) {
                    mine[r] = make_uint4(0u, 0u, 0u, 0u);
                    if (r < S && has_cols && try_load8(silu + ((size_t)r * width) / 2, tag, mine[r])) valid |= 1u << r;
                }
                named_barrier_sync(kConsumerBarrier, kConsumerThreads);  // everybody is done with the previous operand in xbuf
                // The slices' operands are put side by side - two in xbuf, four more in the attention
                // scratch, which no one uses during this phase - so that one barrier serves up to six
                // slices and their tiles are taken back to back (a barrier and a trip through shared
                // memory per slice cost more than the slice's one tile).
                constexpr int kHalves = 6;
                auto half_at = [&](int i) -> bf16 * {
                    return i < 2 ? s.xbuf + i * kChunkCols : reinterpret_cast<bf16 *>(&s.attn[0][0][0]) + (i - 2) * kChunkCols;
                };
                static_assert(sizeof(s.attn) >= (kHalves - 2) * kChunkCols * sizeof(bf16), "attention scratch too small for four operands");
#pragma unroll
                for (int r0 = 0; r0 < kMaxDownSlices; r0 += kHalves) {
                    if (r0 >= S) break;
                    if (r0 > 0) named_barrier_sync(kConsumerBarrier, kConsumerThreads);  // the previous group's operands have been read
#pragma unroll
                    for (int i = 0; i < kHalves; ++i) {
                        const int r = r0 + i;
                        if (r >= kMaxDownSlices || r >= S) break;
                        if (has_cols && !(valid & (1u << r))) load8_wait(p, s, silu + ((size_t)r * width) / 2, tag, mine[r], op, slot + r);
                        if (ctid == 0 && r == 0) stamp(p, slot, kEvDoneWait, t_start);
                        *reinterpret_cast<uint4 *>(&half_at(i)[ctid * 8]) = mine[r];
                    }
                    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
#pragma unroll
                    for (int i = 0; i < kHalves; ++i) {
                        const int r = r0 + i;
                        if (r >= kMaxDownSlices || r >= S) break;
                        if (ctid == 0 && r > 0) stamp(p, slot + r, kEvConsumerStart, t_start);
                        const bf16 *half = half_at(i);
                        uint4 xs[1][8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) xs[0][j] = operand_convert<FP4>(lds128(&half[operand_column<FP4>(cw, t, j)]));
                        if (ctid == 0) stamp(p, slot + r, kEvFirstUse, t_start);
                        for (int b = b0; b < b1; ++b) consume_block<1, FP4>(p, s, st, lane, cw, xs, op, slot + r, 1, width);
                        if (ctid == 0) stamp(p, slot + r, kEvLastUse, t_start);
                    }
                }
                slot += S - 1;  // the slices' instructions have been consumed
                next_ins = after_run;
                continue;
            }
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            // only the gate/up rows of this 2048-column slice have to be ready
            consumer_wait(p, s, ctid, counter(p, layer, kSliceCounterRow, red), p.down_width / kBlockRows, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            uint4 xs[1][8];
            load_operand<1, FP4>(p, s, p.t_silu + ((size_t)layer * p.inter + (size_t)red * p.down_width) / 2, tag, ctid,
                                 p.down_width, xs, op, slot);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<1, FP4>(p, s, st, lane, cw, xs, op, slot, 1, p.down_width);
            break;
        }
        case 7: {
            const int b0 = ins[1], b1 = ins[2];
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, p.layers - 1, 5, 0), p.down_total, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_normed<NCH, FP4>(p, s, ctid, st.norm_toggle, tag, nullptr,
                                  p.t_hidden + (size_t)(p.layers - 1) * (p.hidden / 2), p.lm_norm_w, x, op, slot);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH, FP4>(p, s, st, lane, cw, x, op, slot);
            break;
        }
        default:
            if (ctid == 0) report_failure(p, s, kFailOpcode, op, slot, op, 7);
            break;
        }
        if (ctid == 0) stamp(p, slot, kEvLastUse, t_start);
    }
}

// ---------------------------------------------------------------------------
// storer
// ---------------------------------------------------------------------------

struct StorerState {
    uint32_t pbuf = 0;
    uint32_t pphase = 0;
    __device__ __forceinline__ void advance() {
        if (++pbuf == kPartialBufs) { pbuf = 0; pphase ^= 1u; }
    }
};

// Sum of the 8 consumer warps' partials for row `lane` (lanes 0..15), in warp
// order, then frees the buffer.
__device__ __forceinline__ float collect_block(const Params &p, Smem &s, StorerState &st, int lane, int opcode,
                                               int slot) {
    wait_mbar(p, s, &s.pfull[st.pbuf], st.pphase, kFailPartial, opcode, slot, (int)st.pbuf);
    float v = 0.f;
    if (lane < kBlockRows) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) v += s.partial[st.pbuf][w][lane];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s.pempty[st.pbuf]);
    st.advance();
    return v;
}

// Tells waiting consumers that `value` more blocks exist.  Only a hint (relaxed,
// no fence): the cells themselves carry the launch tag.
__device__ __forceinline__ void publish(const Params &p, Smem &s, int lane, int *ctr, int value) {
    __syncwarp();
    if (lane == 0 && !aborted(s)) red_relaxed_gpu_add(ctr, value);
}

__device__ __forceinline__ unsigned long long argmax_key(float logit_bf16, int index) {
    // Order-preserving map of the bf16 bit pattern; ties resolve to the lowest index.
    uint32_t bits = __float_as_uint(logit_bf16) >> 16;
    bits = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
    return ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (uint32_t)index);
}

// Tensor-parallel all-reduce of a [hidden] vector of fp32 partial sums, issued
// from inside the step: every rank stores its partial of a row into the exchange
// buffer of every GPU (its own included) as a tagged cell, over NVLink for the
// peers; then every rank adds the partials it received in rank order, so all
// ranks compute bit-identical sums without any flag or barrier between GPUs.
__device__ __forceinline__ void tp_push(const Params &p, uint32_t tag, int which, int layer, int row, float v) {
    for (int r = 0; r < p.tp_world; ++r)
        st_tagged_sys(xchg_partials(p, r, tag, which, layer) + (size_t)p.tp_rank * p.hidden + row, __float_as_uint(v), tag);
}

// Receiving side for row blocks b0, b0 + stride, ... below b1: two blocks at a time (lane = block
// parity x row), all ranks' cells in flight at once and retried as a set until
// every tag matches; then residual + bf16(sum) goes to `out` as residual-stream
// cells.  The residual comes from `plain` (layer-0 input) or from `resid` cells.
__device__ void tp_fold_blocks(const Params &p, Smem &s, int lane, uint32_t tag, int which, int layer, int b0, int b1,
                               int stride, const bf16 *plain, const unsigned long long *resid, unsigned long long *out,
                               int op, int slot) {
    const unsigned long long *mine = xchg_partials(p, p.tp_rank, tag, which, layer);
    for (int c0 = b0; c0 < b1; c0 += 2 * stride) {
        const int b = c0 + (lane >> 4) * stride;
        const bool valid = b < b1;
        const int row = (valid ? b : c0) * kBlockRows + (lane & 15);
        unsigned long long v[kMaxRanks];
        unsigned long long rv = 0ull;
        Deadline dl = start_deadline();
        while (true) {
            bool ok = true;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r) {
                v[r] = 0ull;
                if (valid && r < p.tp_world) v[r] = ld_tagged1_sys(mine + (size_t)r * p.hidden + row);
            }
            if (valid && plain == nullptr) rv = ld_tagged1(resid + row / 2);
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (valid && r < p.tp_world) ok &= tag_ok(v[r], tag);
            if (valid && plain == nullptr) ok &= tag_ok(rv, tag);
            if (__all_sync(0xffffffffu, ok) || !keep_waiting(p, s, dl, op, slot, 4)) break;
        }
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.tp_world) total += __uint_as_float(tag_payload(v[r]));
        float h;
        if (plain != nullptr) h = ldcg_bf16(plain + row);
        else h = (row & 1) ? bf16_hi(tag_payload(rv)) : bf16_lo(tag_payload(rv));
        const float o = round_bf16(h + round_bf16(total));
        const float o_next = __shfl_xor_sync(0xffffffffu, o, 1);
        if (valid && (lane & 1) == 0 && !aborted(s)) st_tagged(out + row / 2, pack_bf16x2(o, o_next), tag);
    }
}

// Folds the column slices of down-projection row blocks into the residual
// stream (layer output).  Which blocks an instruction folds:
//   * normally block b belongs to the instruction holding slice (b mod slices) of
//     it, so the work is spread evenly over the SMs; the caller runs this only
//     after the SM has parked all of its own slices of the layer, so the SMs never
//     wait for one another in a cycle;
//   * with p.down_owner_last (queues in which a layer's down-projection
//     instructions are not consecutive) the instruction of the LAST slice folds
//     its blocks right away: it then only waits for slices that precede it in the
//     schedule's dependency order.
// Up to `group` blocks are fetched together, all slices (the SM's own included,
// read back from the cells) with every load in flight at once, and the set is
// retried until every cell carries this launch's tag.  The fold runs in slice
// order: with the interpreter's numerics each slice is rounded to bf16 and added
// with a bf16 rounding (its sequential `hidden += partial`, python_vm.py:59-80);
// with model numerics the slices are summed in fp32, scaled and rounded once.
__device__ void fold_down_blocks(const Params &p, Smem &s, int lane, uint32_t tag, const int *ins, int slot,
                                 long long t_start) {
    const int op = 6;
    const bool writer = lane < kBlockRows, pair_writer = writer && (lane & 1) == 0;
    const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3), red = __ldg(ins + 4);
    const int S = p.down_slices;
    unsigned long long *slice0 = p.t_down + ((size_t)layer * S) * p.hidden;
    int first, step;
    if (p.down_owner_last) {
        first = red == S - 1 ? b0 : b1;
        step = 1;
    } else {
        first = b0 + ((red - b0 % S) % S + S) % S;
        step = S;
    }
    const int group = max(1, min(kDownGroup, (32 * kFetchPerLane) / (kBlockRows * S)));
    for (int g0 = first; g0 < b1; g0 += group * step) {
        const int nb = min(group, (b1 - g0 + step - 1) / step);
        const int ncell = nb * S * kBlockRows;
        unsigned long long pv[kFetchPerLane], rv[kDownGroup];
        Deadline dl = start_deadline();
        while (true) {
            bool ok = true;
#pragma unroll
            for (int j = 0; j < kFetchPerLane; ++j) {
                const int idx = lane + 32 * j;
                if (idx < ncell) {
                    const int i = idx / (S * kBlockRows), rem = idx - i * S * kBlockRows;
                    pv[j] = ld_tagged1(slice0 + (size_t)(rem >> 4) * p.hidden + (g0 + i * step) * kBlockRows + (rem & 15));
                }
            }
#pragma unroll
            for (int i = 0; i < kDownGroup; ++i)
                if (i < nb && pair_writer)
                    rv[i] = ld_tagged1(p.t_resid + ((size_t)layer * p.hidden + (g0 + i * step) * kBlockRows + lane) / 2);
#pragma unroll
            for (int j = 0; j < kFetchPerLane; ++j)
                if (lane + 32 * j < ncell) ok &= tag_ok(pv[j], tag);
#pragma unroll
            for (int i = 0; i < kDownGroup; ++i)
                if (i < nb && pair_writer) ok &= tag_ok(rv[i], tag);
            if (__all_sync(0xffffffffu, ok) || !keep_waiting(p, s, dl, op, slot, 3)) break;
        }
        if (lane == 0) stamp(p, slot, 56, t_start);  // all slices present
#pragma unroll
        for (int j = 0; j < kFetchPerLane; ++j) {
            const int idx = lane + 32 * j;
            if (idx < ncell) {
                const int i = idx / (S * kBlockRows), rem = idx - i * S * kBlockRows;
                s.down_parts[i][rem >> 4][rem & 15] = __uint_as_float(tag_payload(pv[j]));
            }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < kDownGroup; ++i) {
            if (i >= nb) break;
            const int block = g0 + i * step;
            if (p.tp_world > 1) {
                // the local slices are a partial sum over this rank's columns: send it to every rank
                if (writer && !aborted(s)) {
                    float total = 0.f;
                    for (int sl = 0; sl < S; ++sl) total += s.down_parts[i][sl][lane];
                    tp_push(p, tag, 1, layer, block * kBlockRows + lane, total * down_scale(p, layer));
                }
                continue;
            }
            // residual pair (rows lane, lane+1) is held by the even lane
            const uint32_t pr = __shfl_sync(0xffffffffu, tag_payload(rv[i]), lane & ~1);
            float h = (lane & 1) ? bf16_hi(pr) : bf16_lo(pr);
            if (writer) {
                float total = 0.f;
                for (int sl = 0; sl < S; ++sl) {
                    const float part = s.down_parts[i][sl][lane];
                    if (p.model_numerics) total += part;
                    else h = round_bf16(h + round_bf16(part));
                }
                if (p.model_numerics) h = round_bf16(h + round_bf16(total * down_scale(p, layer)));
            }
            const float h_next = __shfl_xor_sync(0xffffffffu, h, 1);
            if (pair_writer && !aborted(s))
                st_tagged(p.t_hidden + ((size_t)layer * p.hidden + block * kBlockRows + lane) / 2, pack_bf16x2(h, h_next), tag);
        }
        __syncwarp();
    }
    if (p.tp_world > 1 && first < b1)
        tp_fold_blocks(p, s, lane, tag, 1, layer, first, b1, step, nullptr, p.t_resid + (size_t)layer * (p.hidden / 2),
                       p.t_hidden + (size_t)layer * (p.hidden / 2), op, slot);
}

template <int NCH>
__device__ void storer_role(const Params &p, Smem &s, int lane, long long t_start) {
    StorerState st;
    const int D = p.hd;
    const int k_start = p.hq * D, v_start = k_start + p.hkv * D;
    const uint32_t tag = __ldg(p.epoch);
    const bf16 *step_input = p.hidden_states;
    if (p.flags & MK_STEP_EMBED) step_input = embedding_row(p);
    const bool writer = lane < kBlockRows;              // lanes that own an output row
    const bool pair_writer = writer && (lane & 1) == 0;  // ... and write the cell of rows (lane, lane+1)
    int run_start = -1, run_layer = -1;                 // consecutive down-projection instructions of one layer

    InsWords next_ins = fetch_instruction(p, 0, lane);
#pragma unroll 1
    for (int slot = 0; slot < p.queue_len; ++slot) {
        const InsWords ins = next_ins;
        next_ins = fetch_instruction(p, slot + 1, lane);  // in flight while this instruction runs
        const int op = ins[0];
        if (op == 0) continue;
        if (lane == 0) stamp(p, slot, kEvStorerStart, t_start);
        switch (op) {
        case 1: {
            // bf16(matvec) -> RoPE in fp32 on Q and K rows -> bf16 store
            // (reference python_vm.py:196-248, llama.py:136-174)
            const int layer = ins[1], b0 = ins[2], b1 = ins[3];
            const size_t cache_row = (((size_t)layer * p.kv_batch) * p.kv_len + p.pos) * (size_t)(p.hkv * D);
            // rotary factors depend only on the position: fetch those of the first
            // two blocks before the sums arrive
            float pre_c[2], pre_s[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int d = ((b0 + i) * kBlockRows + (lane & 15)) % D;
                pre_c[i] = __ldg(p.rope_cos + (size_t)p.pos * D + d);
                pre_s[i] = __ldg(p.rope_sin + (size_t)p.pos * D + d);
            }
            const float ts = matrix_scale(p.q_qkv, layer);
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot) * ts);
                if (lane == 0 && b == b0) stamp(p, slot, kEvFirstStore, t_start);
                const int row = b * kBlockRows + (lane & 15);
                const float other = __shfl_xor_sync(0xffffffffu, y, 1);
                float out = y;
                if (row < v_start) {
                    const int d = row % D;
                    const float c = (b - b0 < 2) ? pre_c[b - b0] : __ldg(p.rope_cos + (size_t)p.pos * D + d);
                    const float sn = (b - b0 < 2) ? pre_s[b - b0] : __ldg(p.rope_sin + (size_t)p.pos * D + d);
                    const float rot = (lane & 1) ? other : -other;
                    out = __fadd_rn(__fmul_rn(y, c), __fmul_rn(rot, sn));
                }
                out = round_bf16(out);
                const float out_next = __shfl_xor_sync(0xffffffffu, out, 1);
                if (writer && !aborted(s)) {
                    const bf16 o = __float2bfloat16_rn(out);
                    // the cache and q buffer serve later launches and the host; this
                    // launch's attention reads the tagged cells
                    unsigned long long *cell;
                    if (row < k_start) {
                        p.q_post[row] = o;
                        cell = p.t_q + ((size_t)layer * k_start + row) / 2;
                    } else if (row < v_start) {
                        p.k_cache[cache_row + (row - k_start)] = o;
                        cell = p.t_k + ((size_t)layer * (v_start - k_start) + (row - k_start)) / 2;
                    } else {
                        p.v_cache[cache_row + (row - v_start)] = o;
                        cell = p.t_v + ((size_t)layer * (v_start - k_start) + (row - v_start)) / 2;
                    }
                    if (pair_writer) st_tagged(cell, pack_bf16x2(out, out_next), tag);
                }
            }
            const int bph = D / kBlockRows;
            __syncwarp();
            if (lane == 0 && !aborted(s)) {
                for (int head = b0 / bph; head <= (b1 - 1) / bph; ++head) {
                    const int lo = max(b0, head * bph), hi = min(b1, (head + 1) * bph);
                    red_relaxed_gpu_add(counter(p, layer, 0, head), hi - lo);
                }
            }
            break;
        }
        case 4: {
            // residual[rows] = bf16(residual[rows] + bf16(matvec)) (reference python_vm.py:59-104)
            const int layer = ins[1], b0 = ins[2], b1 = ins[3];
            // Residual stream entering this layer: the step input or the previous
            // layer's output.  It is upstream of this instruction, so it is fetched
            // (and waited for) before the sums arrive.
            auto residual = [&](int row) {
                if (layer == p.first_layer) return ldcg_bf16(step_input + row);
                const uint32_t pr = load1_wait(p, s, p.t_hidden + ((size_t)(layer - 1) * p.hidden + row) / 2, tag, op, slot);
                return (row & 1) ? bf16_hi(pr) : bf16_lo(pr);
            };
            const float ts = matrix_scale(p.q_o, layer);
            if (p.tp_world > 1) {
                // this rank's columns of the projection are a partial sum: all-reduce, then the residual add
                for (int b = b0; b < b1; ++b) {
                    const float y = collect_block(p, s, st, lane, op, slot) * ts;
                    if (writer && !aborted(s)) tp_push(p, tag, 0, layer, b * kBlockRows + lane, y);
                }
                tp_fold_blocks(p, s, lane, tag, 0, layer, b0, b1, 1, layer == p.first_layer ? step_input : nullptr,
                               p.t_hidden + (size_t)(layer > 0 ? layer - 1 : 0) * (p.hidden / 2),
                               p.t_resid + (size_t)layer * (p.hidden / 2), op, slot);
                publish(p, s, lane, counter(p, layer, 3, 0), b1 - b0);
                break;
            }
            float h = writer ? residual(b0 * kBlockRows + lane) : 0.f;
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot) * ts);
                const float o = round_bf16(h + y);
                const float o_next = __shfl_xor_sync(0xffffffffu, o, 1);
                if (pair_writer && !aborted(s))
                    st_tagged(p.t_resid + ((size_t)layer * p.hidden + b * kBlockRows + lane) / 2, pack_bf16x2(o, o_next), tag);
                if (b + 1 < b1 && writer) h = residual((b + 1) * kBlockRows + lane);
            }
            publish(p, s, lane, counter(p, layer, 3, 0), b1 - b0);
            break;
        }
        case 5: {
            // bf16(bf16(silu(bf16 gate)) * bf16 up) (reference python_vm.py:146-165)
            const int layer = ins[1], n = ins[2];
            const float ts_up = matrix_scale(p.q_up, layer), ts_gate = matrix_scale(p.q_gate, layer);
            for (int i = 0; i < n; ++i) {
                const int b = ins[3 + i];
                const float up = round_bf16(collect_block(p, s, st, lane, op, slot) * ts_up);
                const float gate = round_bf16(collect_block(p, s, st, lane, op, slot) * ts_gate);
                float act = gate / (1.0f + expf(-gate));
                if (!p.model_numerics) act = round_bf16(act);  // the interpreter rounds SiLU before the product
                const float o = round_bf16(act * up);
                const float o_next = __shfl_xor_sync(0xffffffffu, o, 1);
                if (writer && !aborted(s)) {
                    p.silu_out[b * kBlockRows + lane] = __float2bfloat16_rn(o);
                    if (pair_writer)
                        st_tagged(p.t_silu + ((size_t)layer * p.inter + b * kBlockRows + lane) / 2, pack_bf16x2(o, o_next), tag);
                }
            }
            // per 2048-column slice of the product (what one down-projection
            // instruction reads), then the reference interpreter's single counter
            const int listed = ins[(3 + lane) & 31];  // lane i reads list entry i (every lane takes part in the shuffle)
            const int my_slice = lane < n ? (listed * kBlockRows) / p.down_width : -1;
            __syncwarp();
            for (int sl = 0; sl < p.down_slices; ++sl) {
                const int cnt = __popc(__ballot_sync(0xffffffffu, my_slice == sl));
                if (lane == 0 && cnt && !aborted(s)) red_relaxed_gpu_add(counter(p, layer, kSliceCounterRow, sl), cnt);
            }
            if (lane == 0 && !aborted(s)) red_relaxed_gpu_add(counter(p, layer, 4, 0), n);
            break;
        }
        case 6: {
            // fp32 sum over one column slice of a row block, parked per slice as a
            // tagged cell; folding the slices into the residual stream is a separate
            // step (fold_down_blocks), run once this SM has parked all of its slices
            // of the layer.
            const int layer = ins[1], b0 = ins[2], b1 = ins[3], red = ins[4];
            if (p.down_local) {
                // This SM holds every column slice of rows [b0*16, b1*16) as consecutive
                // instructions in slice order, so the interpreter's sequential
                // `hidden += bf16(slice sum)` (python_vm.py:59-80) runs right here: no cells
                // parked for another SM, no second hand-off.  The running value of a row
                // stays in shared memory between the slices' instructions.
                // The run's S instructions are handled here in one go (the queue position
                // moves past them below): one look at the instruction words, the residual
                // fetched once, one counter update.
                const int S = p.down_slices;
                const bool sum_fp32 = p.model_numerics || p.tp_world > 1;  // slices added in fp32, rounded once at the end
                const int nb = b1 - b0;
                // residual entering the MLP block (written by the output projection long ago)
                for (int i = 0; i < nb; ++i) {
                    if (writer && p.tp_world == 1) {
                        const int row = (b0 + i) * kBlockRows + lane;
                        const uint32_t pr = load1_wait(p, s, p.t_resid + ((size_t)layer * p.hidden + row) / 2, tag, op, slot);
                        s.down_acc[i][lane] = (row & 1) ? bf16_hi(pr) : bf16_lo(pr);
                    }
                }
                float total[kLocalBlocks];
#pragma unroll
                for (int i = 0; i < kLocalBlocks; ++i) total[i] = 0.f;
                for (int r = 0; r < S; ++r) {
                    if (lane == 0 && r > 0) stamp(p, slot + r, kEvStorerStart, t_start);
#pragma unroll
                    for (int i = 0; i < kLocalBlocks; ++i) {
                        if (i >= nb) break;
                        const float y = collect_block(p, s, st, lane, op, slot + r);
                        if (writer) {
                            if (sum_fp32) total[i] += y;
                            else s.down_acc[i][lane] = round_bf16(s.down_acc[i][lane] + round_bf16(y));
                        }
                    }
                    if (lane == 0 && r + 1 < S) stamp(p, slot + r, kEvLastStore, t_start);
                }
#pragma unroll
                for (int i = 0; i < kLocalBlocks; ++i) {
                    if (i >= nb) break;
                    const int b = b0 + i;
                    if (p.tp_world > 1) {
                        if (writer && !aborted(s)) tp_push(p, tag, 1, layer, b * kBlockRows + lane, total[i] * down_scale(p, layer));
                        continue;
                    }
                    float h = writer ? s.down_acc[i][lane] : 0.f;
                    if (sum_fp32) h = round_bf16(h + round_bf16(total[i] * down_scale(p, layer)));
                    const float h_next = __shfl_xor_sync(0xffffffffu, h, 1);
                    if (pair_writer && !aborted(s))
                        st_tagged(p.t_hidden + ((size_t)layer * p.hidden + b * kBlockRows + lane) / 2, pack_bf16x2(h, h_next), tag);
                }
                if (p.tp_world > 1)
                    tp_fold_blocks(p, s, lane, tag, 1, layer, b0, b1, 1, nullptr, p.t_resid + (size_t)layer * (p.hidden / 2),
                                   p.t_hidden + (size_t)layer * (p.hidden / 2), op, slot);
                publish(p, s, lane, counter(p, layer, 5, 0), S * nb);  // what the S instructions add together
                slot += S - 1;
                next_ins = fetch_instruction(p, slot + 1, lane);
                if (lane == 0) stamp(p, slot, kEvLastStore, t_start);
                continue;
            }
            unsigned long long *mine = p.t_down + ((size_t)layer * p.down_slices + red) * p.hidden;
            for (int b = b0; b < b1; ++b) {
                const float y = collect_block(p, s, st, lane, op, slot);
                if (writer && !aborted(s)) st_tagged(mine + b * kBlockRows + lane, __float_as_uint(y), tag);
            }
            if (lane == 0) stamp(p, slot, 55, t_start);  // own slices parked
            if (p.down_owner_last) {
                fold_down_blocks(p, s, lane, tag, instruction_at(p, slot), slot, t_start);
            } else {
                if (run_start < 0 || run_layer != layer) { run_start = slot; run_layer = layer; }
                int nxt = slot + 1;
                while (nxt < p.queue_len && __ldg(instruction_at(p, nxt)) == 0) ++nxt;
                const bool more = nxt < p.queue_len && __ldg(instruction_at(p, nxt)) == 6 &&
                                  __ldg(instruction_at(p, nxt) + 1) == layer;
                if (!more) {
                    for (int sl = run_start; sl <= slot; ++sl) {
                        const int *other = instruction_at(p, sl);
                        if (__ldg(other) == 6 && __ldg(other + 1) == layer) fold_down_blocks(p, s, lane, tag, other, slot, t_start);
                    }
                    run_start = -1;
                }
            }
            publish(p, s, lane, counter(p, layer, 5, 0), b1 - b0);
            break;
        }
        case 7: {
            const int b0 = ins[1], b1 = ins[2];
            unsigned long long best = 0ull;
            const float ts = matrix_scale(p.q_lm, 0);
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot) * ts);
                if (lane < kBlockRows && !aborted(s)) {
                    const int row = b * kBlockRows + lane;
                    p.logits[row] = __float2bfloat16_rn(y);
                    const unsigned long long key = argmax_key(y, row);
                    if (key > best) best = key;
                }
            }
#pragma unroll
            for (int off = 8; off; off >>= 1) {
                const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
                if (o > best) best = o;
            }
            if (lane == 0 && best != 0ull && !aborted(s)) atomicMax(p.argmax_key, best);
            break;
        }
        default:
            break;
        }
        if (lane == 0) stamp(p, slot, kEvLastStore, t_start);
    }
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------

template <int NCH, bool FP4>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long t_start = clock64();

    if (tid == 0) {
        for (int i = 0; i < Fmt<FP4>::stages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kConsumerWarps);
        }
        for (int i = 0; i < kPartialBufs; ++i) {
            mbar_init(&s.pfull[i], kConsumerWarps);
            mbar_init(&s.pempty[i], 1);
        }
        // a launch that follows a failed one (status not yet read by the host) does no work: every wait falls through
        s.abort_flag = ld_relaxed_gpu(&p.status[7]) != 0 ? 2 : 0;
        s.is_last = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) loader_role<NCH, FP4>(p, s, t_start);
        __syncwarp();
    } else if (warp < kStorerWarp) {
        consumer_role<NCH, FP4>(p, s, tid - 32, t_start);
    } else {
        storer_role<NCH>(p, s, lane, t_start);
    }

    // ---- last CTA out finishes the step ----
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const int prev = atomicAdd(p.done_counter, 1);
        s.is_last = (prev == (int)gridDim.x - 1);
        __threadfence();
    }
    __syncthreads();
    if (!s.is_last) return;

    // Residual stream handed back to the host: the output of the last layer whose
    // attention block completed - after its MLP block if that completed too.  With
    // no completed block the step input is left as it is.
    const uint32_t tag = __ldg(p.epoch);
    int last = -1;
    for (int l = p.layers - 1; l >= 0; --l) {
        if (ld_relaxed_gpu(counter(p, l, 3, 0)) >= p.hidden / kBlockRows) { last = l; break; }
    }
    if (last >= 0) {
        const bool mlp_done = ld_relaxed_gpu(counter(p, last, 5, 0)) >= p.down_total;
        const unsigned long long *src = (mlp_done ? p.t_hidden : p.t_resid) + (size_t)last * (p.hidden / 2);
        for (int idx = tid; idx < p.hidden; idx += kThreads) {
            const uint32_t pr = tag_payload(ld_tagged1(src + idx / 2));
            p.hidden_states[idx] = __float2bfloat16_rn((idx & 1) ? bf16_hi(pr) : bf16_lo(pr));
        }
    }
    if (tid == 0) *p.epoch = (tag + 1u == 0u) ? 1u : tag + 1u;  // the next launch accepts none of this one's cells
    if (tid == 0) {
        unsigned long long key = __ldcg(p.argmax_key);
        if (p.tp_world > 1 && (p.flags & MK_STEP_WRITE_TOKEN)) {
            // Vocabulary is sharded: send this rank's best (logit bits, global id) to every
            // rank, wait for everybody's, keep the largest key (lowest id on ties).
            if (key) key = (key & 0xffffffff00000000ull) | (unsigned long long)((uint32_t)(key & 0xffffffffull) - (uint32_t)p.vocab_offset);
            for (int r = 0; r < p.tp_world; ++r) {
                unsigned long long *dst = xchg_token(p, r, tag, p.tp_rank);
                st_tagged_sys(dst, (uint32_t)(key >> 32), tag);
                st_tagged_sys(dst + 1, (uint32_t)key, tag);
            }
            unsigned long long best = 0ull;
            Deadline dl = start_deadline();
            for (int r = 0; r < p.tp_world; ++r) {
                const unsigned long long *src = xchg_token(p, p.tp_rank, tag, r);
                unsigned long long hi = ld_tagged1_sys(src), lo = ld_tagged1_sys(src + 1);
                while (!(tag_ok(hi, tag) && tag_ok(lo, tag)) && keep_waiting(p, s, dl, 7, 0, 5)) {
                    hi = ld_tagged1_sys(src);
                    lo = ld_tagged1_sys(src + 1);
                }
                const unsigned long long k = ((unsigned long long)tag_payload(hi) << 32) | tag_payload(lo);
                if (k > best) best = k;
            }
            key = best;
        }
        if ((p.flags & MK_STEP_WRITE_TOKEN) && p.token_out != nullptr)
            *p.token_out = key ? (int)(0xffffffffu - (uint32_t)(key & 0xffffffffull)) : 0;
        *p.argmax_key = 0ull;
        *p.done_counter = 0;
    }
    __syncthreads();
    if (p.flags & MK_STEP_RESET_BARRIERS) {
        const int n = p.layers * p.bar_rows * p.bar_cols;
        for (int i = tid; i < n; i += kThreads) p.bar[i] = 0;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

static thread_local char g_error[512] = "";

static int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

static int cuda_fail(cudaError_t e, const char *what) {
    return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
}

// lets the library's other translation units leave a message for mk_last_error
void set_last_error(const char *msg) { snprintf(g_error, sizeof(g_error), "%s", msg); }

struct Handle {
    MkModelDesc desc;
    Params params;
    int device = 0;
    int nch = 1;
    bool fp4 = false;
    int sm_count = 0;
    int resident = 0;
    cudaFuncAttributes attrs;
    size_t smem_bytes = 0;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // tensor parallelism
    void *xchg = nullptr;              // this GPU's exchange buffer (cudaMalloc, exported over CUDA IPC)
    size_t xchg_bytes = 0;
    int fold_last_detected = 0;        // some queue holds a layer's down-projection instructions apart
    int fold_last_forced = 0;          // MK_OPT_DOWN_FOLD_LAST
    int fold_local_detected = 0;       // every queue keeps the slices of its row blocks together, in order
    int fold_spread_forced = 0;        // MK_OPT_DOWN_FOLD_LOCAL = 0: use the cross-SM fold even where the local one applies
    int plain_launch = 0;              // MK_OPT_COOPERATIVE_LAUNCH = 0: ordinary launch (same grid; co-residency is then the caller's business)
    int tp_world_pending = 0;          // set by mk_tp_init, becomes params.tp_world in mk_tp_connect
    void *peer_xchg[kMaxRanks] = {};   // peers' buffers opened over CUDA IPC
};

static const void *kernel_for(int nch, bool fp4) {
    if (fp4)
        return nch == 2 ? reinterpret_cast<const void *>(&decode_step_kernel<2, true>)
                        : reinterpret_cast<const void *>(&decode_step_kernel<1, true>);
    return nch == 2 ? reinterpret_cast<const void *>(&decode_step_kernel<2, false>)
                    : reinterpret_cast<const void *>(&decode_step_kernel<1, false>);
}

}  // namespace mk

using namespace mk;

extern "C" const char *mk_last_error(void) { return g_error; }

extern "C" int mk_abi_sizeof(int32_t which) {
    switch (which) {
    case 0: return (int)sizeof(MkModelDesc);
    case 1: return (int)sizeof(MkLaunchInfo);
    case 2: return (int)sizeof(MkStatus);
    case 3: return (int)sizeof(MkNvfp4Matrix);
    default: return -1;
    }
}

extern "C" int mk_create(const MkModelDesc *d, void **out) {
    if (!d || !out) return fail(MK_ERR_BAD_ARGUMENT, "mk_create: null argument");
    *out = nullptr;
    if (d->abi_version != MK_ABI_VERSION)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_create: ABI version %d, library has %d", d->abi_version, MK_ABI_VERSION);
    if (d->weight_format != MK_WEIGHTS_BF16 && d->weight_format != MK_WEIGHTS_NVFP4)
        return fail(MK_ERR_UNSUPPORTED, "mk_create: weight format %d not supported by this build", d->weight_format);
    const bool fp4 = d->weight_format == MK_WEIGHTS_NVFP4;
    const int H = d->hidden_size, D = d->head_dim;
    if (H <= 0 || d->num_layers <= 0 || d->num_q_heads <= 0 || d->num_kv_heads <= 0 || D <= 0 ||
        d->intermediate_size <= 0 || d->vocab_size <= 0)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_create: non-positive dimension");
    if (H != kChunkCols && H != 2 * kChunkCols)
        return fail(MK_ERR_UNSUPPORTED, "hidden_size %d: kernel streams 2048-column tiles, hidden must be 2048 or 4096", H);
    // Input width of the output projection: hidden_size for a whole model, a 1/n
    // share of it for a tensor-parallel rank.
    const int o_cols = d->num_q_heads * D;
    if (o_cols > H || (o_cols >= kChunkCols ? o_cols % kChunkCols != 0 : o_cols % 256 != 0))
        return fail(MK_ERR_UNSUPPORTED, "num_q_heads*head_dim = %d: must be a multiple of 2048 up to hidden_size, or a multiple of 256 below 2048", o_cols);
    if (D != 64 && D != 128) return fail(MK_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", D);
    if (d->num_q_heads != kGroup * d->num_kv_heads)
        return fail(MK_ERR_UNSUPPORTED, "query group size must be %d (got %d q heads, %d kv heads)", kGroup, d->num_q_heads, d->num_kv_heads);
    // Down-projection column slices: the widest multiple of 256 up to 2048 that divides
    // intermediate_size (2048 for whole models; e.g. 1792 for 14336/2, /4 and /8).
    int down_width = 0;
    for (int w = kChunkCols; w >= 256; w -= 256)
        if (d->intermediate_size % w == 0) { down_width = w; break; }
    if (!down_width) return fail(MK_ERR_UNSUPPORTED, "intermediate_size %d not a multiple of 256", d->intermediate_size);
    if (d->vocab_size % kBlockRows) return fail(MK_ERR_UNSUPPORTED, "vocab_size %d not a multiple of 16", d->vocab_size);
    if (d->barrier_rows < 8 || d->barrier_cols < d->num_q_heads + 2 * d->num_kv_heads)
        return fail(MK_ERR_BAD_ARGUMENT, "barriers tensor too small: rows %d cols %d", d->barrier_rows, d->barrier_cols);
    if (d->kv_batch < 1 || d->kv_max_len < 1 || d->rope_positions < 1 || d->max_partials < 1)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_create: cache/rope/partials extent must be positive");
    if (fp4) {
        const MkNvfp4Matrix *tables[] = {d->qkv_q, d->o_q, d->up_q, d->gate_q, d->down_q, d->lm_head_q};
        for (int ti = 0; ti < 6; ++ti) {
            if (!tables[ti]) return fail(MK_ERR_BAD_ARGUMENT, "mk_create: NVFP4 model without a quantised weight table");
            const int count = ti == 5 ? 1 : d->num_layers;
            for (int i = 0; i < count; ++i) {
                const MkNvfp4Matrix &q = tables[ti][i];
                if (!q.packed || !q.scales || (reinterpret_cast<uintptr_t>(q.packed) & 15) ||
                    (reinterpret_cast<uintptr_t>(q.scales) & 15) || !(q.tensor_scale > 0.f))
                    return fail(MK_ERR_BAD_ARGUMENT, "mk_create: NVFP4 matrix %d/%d: null or misaligned pointer, or non-positive scale", ti, i);
            }
        }
    } else {
        const void *weights[] = {d->qkv_w, d->o_w, d->up_w, d->gate_w, d->down_w, d->lm_head_w};
        for (const void *ptr : weights)
            if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 15))
                return fail(MK_ERR_BAD_ARGUMENT, "mk_create: null or misaligned bf16 weight pointer");
    }
    const void *required[] = {d->attn_norm_w,
                              d->mlp_norm_w, d->lm_head_norm_w, d->k_cache, d->v_cache, d->rope_cos, d->rope_sin,
                              d->hidden_states, d->q_post_rope, d->attn_out, d->attn_lse_intermediates,
                              d->attn_out_intermediates, d->silu_out, d->logits, d->barriers};
    for (const void *ptr : required) {
        if (!ptr) return fail(MK_ERR_BAD_ARGUMENT, "mk_create: null device pointer in descriptor");
        if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(MK_ERR_BAD_ARGUMENT, "mk_create: device pointer %p not 16-byte aligned", ptr);
    }

    Handle *h = new (std::nothrow) Handle();
    if (!h) return fail(MK_ERR_BAD_ARGUMENT, "mk_create: out of host memory");
    h->desc = *d;
    h->nch = H / kChunkCols;
    h->fp4 = fp4;
    cudaError_t e = cudaGetDevice(&h->device);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaGetDevice"); }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, h->device);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaGetDeviceProperties"); }
    h->sm_count = prop.multiProcessorCount;
    if (!prop.cooperativeLaunch) { delete h; return fail(MK_ERR_RESIDENCY, "device does not support cooperative launch"); }

    const void *kern = kernel_for(h->nch, h->fp4);
    h->smem_bytes = sizeof(Smem) + 128;
    int optin = 0;
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, h->device);
    e = cudaFuncGetAttributes(&h->attrs, kern);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaFuncGetAttributes (is this an sm_100a device?)"); }
    if (h->smem_bytes + h->attrs.sharedSizeBytes > (size_t)optin) {
        delete h;
        return fail(MK_ERR_RESIDENCY, "shared memory %zu + %zu exceeds the device opt-in limit %d", h->smem_bytes, h->attrs.sharedSizeBytes, optin);
    }
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)h->smem_bytes);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaFuncSetAttribute"); }
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&h->resident, kern, kThreads, h->smem_bytes);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "occupancy query"); }
    if (h->resident < 1) { delete h; return fail(MK_ERR_RESIDENCY, "kernel cannot keep one CTA resident per SM"); }

    // scratch: tagged cells | argmax key (8 B) | exit counter | status[8] | launch tag
    const int slices = d->intermediate_size / down_width;
    if (slices > kMaxDownSlices) { delete h; return fail(MK_ERR_UNSUPPORTED, "intermediate_size %d: at most %d column slices", d->intermediate_size, kMaxDownSlices); }
    const size_t L = d->num_layers, qd = (size_t)d->num_q_heads * D, kvd = (size_t)d->num_kv_heads * D;
    const size_t n_resid = L * H / 2, n_hidden = L * H / 2, n_down = L * slices * H, n_q = L * qd / 2, n_kv = L * kvd / 2, n_attn = L * qd / 2;
    const size_t n_silu = L * d->intermediate_size / 2, n_oi = L * d->num_q_heads * kTaggedPartials * D;
    const size_t n_lse = L * d->num_q_heads * kTaggedPartials;
    const size_t cells = n_resid + n_hidden + n_down + n_q + 2 * n_kv + n_attn + n_silu + n_oi + n_lse;
    const size_t cell_bytes = (cells * sizeof(unsigned long long) + 255) & ~size_t(255);
    const size_t table_entries = fp4 ? 5 * L + 1 : 0;  // device copies of the quantised-matrix tables
    const size_t table_bytes = (table_entries * sizeof(MkNvfp4Matrix) + 255) & ~size_t(255);
    const size_t stuck_bytes = (size_t)h->sm_count * (kThreads / 32) * 4 * sizeof(int);
    h->scratch_bytes = cell_bytes + 256 + table_bytes + stuck_bytes;
    e = cudaMalloc(&h->scratch, h->scratch_bytes);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaMalloc(scratch)"); }
    e = cudaMemset(h->scratch, 0, h->scratch_bytes);  // tag 0 is never a launch tag
    if (e != cudaSuccess) { cudaFree(h->scratch); delete h; return cuda_fail(e, "cudaMemset(scratch)"); }
    const unsigned first_tag = 1;
    e = cudaMemcpy((uint8_t *)h->scratch + cell_bytes + 64, &first_tag, sizeof(first_tag), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(h->scratch); delete h; return cuda_fail(e, "cudaMemcpy(launch tag)"); }

    Params &p = h->params;
    memset(&p, 0, sizeof(p));
    p.hidden = H; p.layers = d->num_layers; p.hq = d->num_q_heads; p.hkv = d->num_kv_heads; p.hd = D;
    p.inter = d->intermediate_size; p.vocab = d->vocab_size;
    p.qkv_rows = (d->num_q_heads + 2 * d->num_kv_heads) * D;
    p.kv_batch = d->kv_batch; p.kv_len = d->kv_max_len;
    p.max_partials = d->max_partials;
    p.bar_rows = d->barrier_rows; p.bar_cols = d->barrier_cols;
    p.skip_attn_reduction = d->skip_attn_reduction;
    p.attn_scale = d->attn_scale; p.eps = d->rms_norm_eps;
    p.spin_cycles = 4000000000ll;
    p.early_shift = 0;
    p.max_inflight = kMaxStages;
    p.o_cols = o_cols;
    p.o_chunks = o_cols >= kChunkCols ? o_cols / kChunkCols : 1;
    p.o_width = o_cols >= kChunkCols ? kChunkCols : o_cols;
    p.down_width = down_width;
    p.down_slices = slices;
    p.down_total = (H / kBlockRows) * slices;
    p.qkv_w = (const bf16 *)d->qkv_w; p.attn_norm_w = (const bf16 *)d->attn_norm_w; p.o_w = (const bf16 *)d->o_w;
    p.mlp_norm_w = (const bf16 *)d->mlp_norm_w; p.up_w = (const bf16 *)d->up_w; p.gate_w = (const bf16 *)d->gate_w;
    p.down_w = (const bf16 *)d->down_w; p.lm_norm_w = (const bf16 *)d->lm_head_norm_w; p.lm_w = (const bf16 *)d->lm_head_w;
    p.embed_w = (const bf16 *)d->embed_w;
    p.k_cache = (bf16 *)d->k_cache; p.v_cache = (bf16 *)d->v_cache;
    p.rope_cos = d->rope_cos; p.rope_sin = d->rope_sin;
    p.hidden_states = (bf16 *)d->hidden_states; p.q_post = (bf16 *)d->q_post_rope; p.attn_out = (bf16 *)d->attn_out;
    p.attn_lse = d->attn_lse_intermediates; p.attn_oi = d->attn_out_intermediates;
    p.silu_out = (bf16 *)d->silu_out; p.logits = (bf16 *)d->logits;
    p.bar = d->barriers;
    uint8_t *sc = (uint8_t *)h->scratch;
    unsigned long long *cell = (unsigned long long *)sc;
    p.t_resid = cell; cell += n_resid;
    p.t_hidden = cell; cell += n_hidden;
    p.t_down = cell;  cell += n_down;
    p.t_q = cell;     cell += n_q;
    p.t_k = cell;     cell += n_kv;
    p.t_v = cell;     cell += n_kv;
    p.t_attn = cell;  cell += n_attn;
    p.t_silu = cell;  cell += n_silu;
    p.t_oi = cell;    cell += n_oi;
    p.t_lse = cell;   cell += n_lse;
    p.argmax_key = (unsigned long long *)(sc + cell_bytes);
    p.done_counter = (int *)(sc + cell_bytes + 16);
    p.status = (int *)(sc + cell_bytes + 32);
    p.epoch = (unsigned *)(sc + cell_bytes + 64);
    p.stuck = (int *)(sc + cell_bytes + 256 + table_bytes);
    p.model_numerics = fp4 ? 1 : 0;
    p.tp_rank = 0; p.tp_world = 1; p.vocab_offset = 0;
    if (fp4) {
        MkNvfp4Matrix *dev = (MkNvfp4Matrix *)(sc + cell_bytes + 256);
        const MkNvfp4Matrix *src[] = {d->qkv_q, d->o_q, d->up_q, d->gate_q, d->down_q};
        const MkNvfp4Matrix **dst[] = {&p.q_qkv, &p.q_o, &p.q_up, &p.q_gate, &p.q_down};
        for (int ti = 0; ti < 5; ++ti) {
            e = cudaMemcpy(dev + ti * L, src[ti], L * sizeof(MkNvfp4Matrix), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) { cudaFree(h->scratch); delete h; return cuda_fail(e, "cudaMemcpy(weight table)"); }
            *dst[ti] = dev + ti * L;
        }
        e = cudaMemcpy(dev + 5 * L, d->lm_head_q, sizeof(MkNvfp4Matrix), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { cudaFree(h->scratch); delete h; return cuda_fail(e, "cudaMemcpy(weight table)"); }
        p.q_lm = dev + 5 * L;
    }
    *out = h;
    return 0;
}

extern "C" int mk_set_schedule(void *handle, const int32_t *instructions, int32_t *timings, int32_t workers,
                               int32_t queue_len) {
    Handle *h = (Handle *)handle;
    if (!h) return fail(MK_ERR_BAD_ARGUMENT, "mk_set_schedule: null handle");
    if (workers <= 0 || queue_len < 0 || (!instructions && queue_len > 0))
        return fail(MK_ERR_BAD_ARGUMENT, "mk_set_schedule: bad queue dimensions %d x %d", workers, queue_len);
    if (workers > h->sm_count * h->resident)
        return fail(MK_ERR_RESIDENCY, "worker grid (%d) exceeds co-resident capacity (%d SMs x %d)", workers, h->sm_count, h->resident);
    if (workers > h->sm_count)
        return fail(MK_ERR_RESIDENCY, "worker grid (%d) exceeds the physical SM count (%d)", workers, h->sm_count);
    // The queues are read once on the host.  Every operand the device uses as an
    // index is checked here, so that a hand-built instruction tensor is refused
    // before anything launches instead of writing outside the handle's buffers.
    //
    // Down-projection folding mode (fold_down_blocks): spreading the folds over all
    // SMs needs every queue to hold a layer's down-projection instructions (opcode 6)
    // consecutively, which the reference's assignment policies all produce.  Any
    // other ordering gets the mode in which only the last slice's instruction folds.
    int owner_last = 0;
    int first_layer = 0;
    int local = 0;
    if (queue_len > 0) {
        const size_t words = (size_t)workers * queue_len * kInstrWords;
        int32_t *host = new (std::nothrow) int32_t[words];
        if (!host) return fail(MK_ERR_BAD_ARGUMENT, "mk_set_schedule: out of host memory");
        cudaError_t e = cudaMemcpy(host, instructions, words * sizeof(int32_t), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { delete[] host; return cuda_fail(e, "cudaMemcpy(instructions)"); }
        const Params &p = h->params;
        const int slots = p.max_partials < kTaggedPartials ? p.max_partials : kTaggedPartials;  // attention slices addressable
        const int hidden_blocks = p.hidden / kBlockRows;
        int lowest = p.layers;
        for (int w = 0; w < workers; ++w) {
            for (int q = 0; q < queue_len; ++q) {
                const int32_t *ins = host + ((size_t)w * queue_len + q) * kInstrWords;
                const int op = ins[0];
                const char *why = nullptr;
                auto blocks_ok = [](int b0, int b1, int limit) { return 0 <= b0 && b0 <= b1 && b1 <= limit; };
                if (op == 0) continue;
                if (op < 0 || op > 7) why = "opcode outside 0..7";
                else if (op != 7 && (ins[1] < 0 || ins[1] >= p.layers)) why = "layer outside the model";
                else if (op == 1 && !blocks_ok(ins[2], ins[3], p.qkv_rows / kBlockRows)) why = "QKV row blocks outside the matrix";
                else if (op == 2 && (ins[2] < 0 || ins[2] >= p.hkv)) why = "KV head outside the model";
                else if (op == 2 && (ins[3] < 1 || ins[3] > slots || ins[4] < 0 || ins[4] >= ins[3])) why = "attention slice outside 0..min(32, max_partials)";
                else if (op == 3 && (ins[2] < 0 || ins[2] + kGroup > p.hq)) why = "query heads outside the model";
                else if (op == 3 && (ins[5] < 1 || 6 + ins[5] + 1 > kInstrWords)) why = "reduction list does not fit the instruction";
                else if ((op == 4 || op == 6) && !blocks_ok(ins[2], ins[3], hidden_blocks)) why = "output row blocks outside the matrix";
                else if (op == 6 && (ins[4] < 0 || ins[4] >= p.down_slices)) why = "column slice outside the down projection";
                else if (op == 5 && (ins[2] < 0 || 3 + ins[2] > kInstrWords)) why = "block list does not fit the instruction";
                else if (op == 7 && !blocks_ok(ins[1], ins[2], p.vocab / kBlockRows)) why = "vocabulary row blocks outside the matrix";
                if (!why && op == 3) {
                    for (int j = 0; j < ins[5]; ++j)
                        if (ins[6 + j] < 0 || ins[6 + j] >= slots) why = "reduction list entry outside 0..min(32, max_partials)";
                    if (!ins[4] && (ins[6 + ins[5]] < 0 || ins[6 + ins[5]] >= slots)) why = "output slice outside 0..min(32, max_partials)";
                }
                if (!why && op == 5) {
                    for (int j = 0; j < ins[2]; ++j)
                        if (ins[3 + j] < 0 || ins[3 + j] >= p.inter / kBlockRows) why = "gate/up row block outside the matrix";
                }
                if (why) {
                    delete[] host;
                    return fail(MK_ERR_BAD_ARGUMENT, "mk_set_schedule: worker %d slot %d opcode %d: %s", w, q, op, why);
                }
                if (op != 7 && ins[1] < lowest) lowest = ins[1];
            }
        }
        first_layer = lowest < p.layers ? lowest : 0;
        // Local folding: every queue holds the column slices of its down-projection row
        // blocks as consecutive instructions (no-ops aside) in slice order 0..S-1.
        local = 1;
        for (int w = 0; w < workers && local; ++w) {
            int expect = 0, layer = -1, b0 = -1, b1 = -1;  // next slice expected within the current run
            for (int q = 0; q < queue_len && local; ++q) {
                const int32_t *ins = host + ((size_t)w * queue_len + q) * kInstrWords;
                if (ins[0] != 6) { if (expect != 0) local = 0; continue; }  // a run has no gaps, not even no-ops
                if (expect == 0) { layer = ins[1]; b0 = ins[2]; b1 = ins[3]; }
                if (ins[1] != layer || ins[2] != b0 || ins[3] != b1 || ins[4] != expect || b1 - b0 > kLocalBlocks) local = 0;
                expect = (expect + 1) % p.down_slices;
            }
            if (expect != 0) local = 0;
        }
        for (int w = 0; w < workers && !owner_last; ++w) {
            int run_layer = -1;            // layer of the run of opcode-6 instructions being read, -1 outside a run
            unsigned long long seen = 0;   // layers whose run has ended (layers >= 64 fall back at once)
            for (int q = 0; q < queue_len; ++q) {
                const int32_t *ins = host + ((size_t)w * queue_len + q) * kInstrWords;
                if (ins[0] == 0) continue;
                const int layer = ins[0] == 6 ? ins[1] : -1;
                if (layer != run_layer) {
                    if (run_layer >= 0) seen |= 1ull << run_layer;
                    run_layer = layer;
                    if (layer >= 64 || (layer >= 0 && (seen >> layer) & 1ull)) { owner_last = 1; break; }
                }
            }
        }
        delete[] host;
    }
    h->params.first_layer = first_layer;
    h->fold_local_detected = local;
    h->params.down_local = local && !h->fold_last_forced && !h->fold_spread_forced;
    h->fold_last_detected = owner_last;
    h->params.down_owner_last = owner_last || h->fold_last_forced;
    h->params.instructions = instructions;
    h->params.timings = timings;
    h->params.workers = workers;
    h->params.queue_len = queue_len;
    return 0;
}

extern "C" int mk_step(void *handle, int32_t pos_id, uint32_t flags, const int32_t *token_in, int32_t *token_out,
                       void *stream) {
    Handle *h = (Handle *)handle;
    if (!h) return fail(MK_ERR_BAD_ARGUMENT, "mk_step: null handle");
    Params p = h->params;
    if (p.workers <= 0) return fail(MK_ERR_BAD_ARGUMENT, "mk_step: no schedule attached (call mk_set_schedule)");
    if (pos_id < 0 || pos_id >= h->desc.kv_max_len || pos_id >= h->desc.rope_positions)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_step: pos_id %d outside cache (%d) or rope table (%d)", pos_id, h->desc.kv_max_len, h->desc.rope_positions);
    if ((flags & MK_STEP_EMBED) && (!p.embed_w || !token_in))
        return fail(MK_ERR_BAD_ARGUMENT, "mk_step: MK_STEP_EMBED needs embed_w in the descriptor and a token_in pointer");
    if ((flags & MK_STEP_WRITE_TOKEN) && !token_out)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_step: MK_STEP_WRITE_TOKEN needs a token_out pointer");
    if ((flags & MK_STEP_TIMINGS) && !p.timings)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_step: MK_STEP_TIMINGS needs a timings tensor");
    if (p.queue_len == 0) return 0;
    p.pos = pos_id;
    p.flags = flags;
    p.token_in = token_in;
    p.token_out = token_out;
    void *args[] = {&p};
    cudaError_t e = h->plain_launch
                        ? cudaLaunchKernel(kernel_for(h->nch, h->fp4), dim3(p.workers), dim3(kThreads), args, h->smem_bytes,
                                           (cudaStream_t)stream)
                        : cudaLaunchCooperativeKernel(kernel_for(h->nch, h->fp4), dim3(p.workers), dim3(kThreads), args,
                                                      h->smem_bytes, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cooperative megakernel launch");
    return 0;
}

extern "C" int mk_query(void *handle, MkLaunchInfo *info) {
    Handle *h = (Handle *)handle;
    if (!h || !info) return fail(MK_ERR_BAD_ARGUMENT, "mk_query: null argument");
    memset(info, 0, sizeof(*info));
    info->cooperative_launch = 1;
    info->physical_sms = h->sm_count;
    info->resident_worker_capacity = h->sm_count * h->resident;
    info->active_workers = h->params.workers;
    info->threads_per_cta = kThreads;
    info->consumer_warps = kConsumerWarps;
    info->registers_per_thread = h->attrs.numRegs;
    info->local_bytes_per_thread = (int)h->attrs.localSizeBytes;
    info->static_smem_bytes = (int)h->attrs.sharedSizeBytes;
    info->dynamic_smem_bytes = (int)h->smem_bytes;
    info->stage_count = h->fp4 ? kFp4Stages : kStages;
    info->stage_bytes = h->fp4 ? kFp4TileBytes : kStageBytes;
    info->resident_ctas_per_sm = h->resident;
    info->queue_len = h->params.queue_len;
    info->scratch_bytes = (int64_t)h->scratch_bytes;
    info->down_fold_mode = h->params.down_local ? 2 : (h->params.down_owner_last ? 1 : 0);
    return 0;
}

extern "C" int mk_status(void *handle, MkStatus *status, void *stream) {
    Handle *h = (Handle *)handle;
    if (!h) return fail(MK_ERR_BAD_ARGUMENT, "mk_status: null handle");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    int words[8];
    e = cudaMemcpy(words, h->params.status, sizeof(words), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
    if (status) {
        status->code = words[0]; status->worker = words[1]; status->opcode = words[2];
        status->slot = words[3]; status->detail = words[4]; status->expected = words[5];
    }
    if (words[0] != 0 || words[7] != 0) {
        // leave the handle reusable: clear status, argmax cell and the exit counter
        cudaMemset(h->params.argmax_key, 0, 64);
        return fail(MK_ERR_DEVICE_WAIT, "device wait expired: code %d worker %d opcode %d slot %d saw %d expected %d",
                    words[0], words[1], words[2], words[3], words[4], words[5]);
    }
    return 0;
}

extern "C" int mk_status_detail(void *handle, int32_t *records, int32_t max_records, int32_t *count) {
    Handle *h = (Handle *)handle;
    if (!h || !records || max_records < 0 || !count) return fail(MK_ERR_BAD_ARGUMENT, "mk_status_detail: bad argument");
    const int warps = kThreads / 32, total = h->sm_count * warps;
    int32_t *all = new (std::nothrow) int32_t[(size_t)total * 4];
    if (!all) return fail(MK_ERR_BAD_ARGUMENT, "mk_status_detail: out of host memory");
    cudaError_t e = cudaMemcpy(all, h->params.stuck, (size_t)total * 4 * sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemset(h->params.stuck, 0, (size_t)total * 4 * sizeof(int32_t));
    if (e != cudaSuccess) { delete[] all; return cuda_fail(e, "mk_status_detail"); }
    int n = 0;
    for (int i = 0; i < total; ++i) {
        if (all[4 * i] == 0) continue;
        if (n < max_records) {
            int32_t *r = records + 6 * n;
            r[0] = i / warps; r[1] = i % warps; r[2] = all[4 * i]; r[3] = all[4 * i + 1]; r[4] = all[4 * i + 2]; r[5] = all[4 * i + 3];
        }
        ++n;
    }
    delete[] all;
    *count = n;
    return 0;
}

extern "C" int mk_set_wait_budget(void *handle, int64_t cycles) {
    Handle *h = (Handle *)handle;
    if (!h || cycles <= 0) return fail(MK_ERR_BAD_ARGUMENT, "mk_set_wait_budget: bad argument");
    h->params.spin_cycles = cycles;
    return 0;
}

extern "C" int mk_set_option(void *handle, int32_t option, int64_t value) {
    Handle *h = (Handle *)handle;
    if (!h) return fail(MK_ERR_BAD_ARGUMENT, "mk_set_option: null handle");
    switch (option) {
    case MK_OPT_WAIT_BUDGET_CYCLES:
        if (value <= 0) return fail(MK_ERR_BAD_ARGUMENT, "wait budget must be positive");
        h->params.spin_cycles = value;
        return 0;
    case MK_OPT_MAX_INFLIGHT_TILES:
        if (value < 1) return fail(MK_ERR_BAD_ARGUMENT, "at least one tile must be in flight");
        h->params.max_inflight = (int)(value > kMaxStages ? kMaxStages : value);
        return 0;
    case MK_OPT_DOWN_FOLD_LAST:
        h->fold_last_forced = value != 0;
        h->params.down_owner_last = h->fold_last_detected || h->fold_last_forced;
        h->params.down_local = h->fold_local_detected && !h->fold_last_forced && !h->fold_spread_forced;
        return 0;
    case MK_OPT_DOWN_FOLD_LOCAL:
        h->fold_spread_forced = value == 0;
        h->params.down_local = h->fold_local_detected && !h->fold_last_forced && !h->fold_spread_forced;
        return 0;
    case MK_OPT_COOPERATIVE_LAUNCH:
        h->plain_launch = value == 0;
        return 0;
    case MK_OPT_EARLY_POLL_SHIFT:
        if (value < 0 || value > 31) return fail(MK_ERR_BAD_ARGUMENT, "early-poll shift must be 0..31");
        h->params.early_shift = (int)value;
        return 0;
    default:
        return fail(MK_ERR_BAD_ARGUMENT, "mk_set_option: unknown option %d", option);
    }
}

extern "C" int mk_tp_init(void *handle, int32_t rank, int32_t world, int32_t vocab_offset, void *ipc_handle_out) {
    Handle *h = (Handle *)handle;
    if (!h || !ipc_handle_out) return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_init: null argument");
    if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world || vocab_offset < 0)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_init: rank %d of %d (2..%d ranks), vocabulary offset %d", rank, world, kMaxRanks, vocab_offset);
    if (h->xchg) return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_init: already initialised");
    static_assert(sizeof(cudaIpcMemHandle_t) == MK_TP_HANDLE_BYTES, "IPC handle size");
    const Params &p = h->params;
    const size_t cells = (size_t)2 * 2 * p.layers * world * p.hidden + (size_t)2 * world * 2;
    h->xchg_bytes = cells * sizeof(unsigned long long);
    cudaError_t e = cudaSetDevice(h->device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    e = cudaMalloc(&h->xchg, h->xchg_bytes);
    if (e != cudaSuccess) { h->xchg = nullptr; return cuda_fail(e, "cudaMalloc(exchange buffer)"); }
    e = cudaMemset(h->xchg, 0, h->xchg_bytes);  // tag 0 is never a launch tag
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaIpcGetMemHandle((cudaIpcMemHandle_t *)ipc_handle_out, h->xchg);
    if (e != cudaSuccess) { cudaFree(h->xchg); h->xchg = nullptr; return cuda_fail(e, "exchange buffer set-up"); }
    h->params.tp_rank = rank;
    h->params.vocab_offset = vocab_offset;
    h->tp_world_pending = world;
    return 0;
}

extern "C" int mk_tp_connect(void *handle, const void *ipc_handles, int32_t count) {
    Handle *h = (Handle *)handle;
    if (!h || !ipc_handles) return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_connect: null argument");
    if (!h->xchg || h->tp_world_pending < 2) return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_connect: call mk_tp_init first");
    if (h->params.tp_world > 1) return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_connect: already connected");
    if (count != h->tp_world_pending)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_tp_connect: %d handles given, mk_tp_init was told %d ranks", count, h->tp_world_pending);
    cudaError_t e = cudaSetDevice(h->device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    // Steps made on this handle before connecting (a single-GPU warm-up) left cells
    // tagged 1, 2, ...; the launch count restarts at 1 below, so those cells are
    // cleared: no launch after the restart may accept one of them as its own.
    e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemset(h->scratch, 0, (size_t)((uint8_t *)h->params.argmax_key - (uint8_t *)h->scratch));
    if (e != cudaSuccess) return cuda_fail(e, "clearing the hand-off cells");
    const cudaIpcMemHandle_t *handles = (const cudaIpcMemHandle_t *)ipc_handles;
    for (int r = 0; r < h->tp_world_pending; ++r) {
        if (r == h->params.tp_rank) {
            h->params.xchg[r] = (unsigned long long *)h->xchg;
            continue;
        }
        void *ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, handles[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle (are all ranks on one NVLink-connected node, one process per GPU?)");
        h->peer_xchg[r] = ptr;
        h->params.xchg[r] = (unsigned long long *)ptr;
    }
    // every rank starts counting launches from the same tag
    const unsigned first_tag = 1;
    e = cudaMemcpy(h->params.epoch, &first_tag, sizeof(first_tag), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(launch tag)");
    h->params.tp_world = h->tp_world_pending;
    return 0;
}

extern "C" void mk_destroy(void *handle) {
    Handle *h = (Handle *)handle;
    if (!h) return;
    for (int r = 0; r < kMaxRanks; ++r)
        if (h->peer_xchg[r]) cudaIpcCloseMemHandle(h->peer_xchg[r]);
    if (h->xchg) cudaFree(h->xchg);
    cudaFree(h->scratch);
    delete h;
}
