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
constexpr int kStages = 3;                                // tiles in flight per SM (192 KiB)
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

// timing slots (reference include/util.cuh:225-256)
constexpr int kEvLoaderStart = 5, kEvStorerStart = 9, kEvConsumerStart = 11;
constexpr int kEvAtWait = 44, kEvDoneWait = 45, kEvFirstLoad = 48, kEvFirstUse = 49, kEvFirstStore = 50;
constexpr int kEvLastLoad = 51, kEvLastUse = 52, kEvLastStore = 53, kEvOutputReady = 54;

// status codes
constexpr int kFailCounter = 1, kFailRing = 2, kFailPartial = 3, kFailOpcode = 4;

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
    int down_slices;  // inter / 2048
    int down_total;   // (hidden / 16) * down_slices
    // weights
    const bf16 *qkv_w, *attn_norm_w, *o_w, *mlp_norm_w, *up_w, *gate_w, *down_w, *lm_norm_w, *lm_w, *embed_w;
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
    bf16 *down_partials;            // [down_slices][hidden]
    unsigned long long *argmax_key;
    int *done_counter;
    int *status;                    // [0] code [1] worker [2] opcode [3] slot [4] detail [5] expected [7] abort
    const int *token_in;
    int *token_out;
};

struct __align__(128) Smem {
    uint8_t stage[kStages][kStageBytes];
    float attn[kConsumerWarps][kGroup][kMaxHeadDim + 2];
    float partial[kPartialBufs][kConsumerWarps][kBlockRows];
    float red[2][kConsumerWarps];
    __align__(16) bf16 xbuf[2 * kChunkCols];  // normalised activations, re-read in the MMA operand layout
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t pfull[kPartialBufs];
    uint64_t pempty[kPartialBufs];
    int abort_flag;
    int is_last;
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------

__device__ __forceinline__ bool aborted(const Smem &s) { return *reinterpret_cast<const volatile int *>(&s.abort_flag) != 0; }

__device__ __noinline__ void report_failure(const Params &p, Smem &s, int code, int opcode, int slot, int detail,
                                            int expected) {
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
            if (aborted(s)) return;
            if ((it & 1023u) == 0 && ld_relaxed_gpu(&p.status[7]) != 0) {
                *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
                return;
            }
            if (clock64() - t0 > p.spin_cycles) {
                report_failure(p, s, code, opcode, slot, detail, (int)parity);
                return;
            }
        }
    }
}

// One thread polls a dependency counter until it reaches `expected`.
__device__ __forceinline__ void wait_counter(const Params &p, Smem &s, const int *ctr, int expected, int opcode,
                                             int slot) {
    if (aborted(s)) return;
    int v = ld_acquire_gpu(ctr);
    if (v >= expected) return;
    const long long t0 = clock64();
    unsigned it = 0;
    while (true) {
        __nanosleep(20);
        v = ld_acquire_gpu(ctr);
        if (v >= expected) return;
        if ((++it & 15u) == 0) {
            if (aborted(s)) return;
            if (ld_relaxed_gpu(&p.status[7]) != 0) {
                *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
                return;
            }
            if (clock64() - t0 > p.spin_cycles) {
                report_failure(p, s, kFailCounter, opcode, slot, v, expected);
                return;
            }
        }
    }
}

__device__ __forceinline__ int *counter(const Params &p, int layer, int row, int col) {
    return p.bar + ((size_t)layer * p.bar_rows + row) * p.bar_cols + col;
}

__device__ __forceinline__ const int *instruction_at(const Params &p, int slot) {
    return p.instructions + ((size_t)blockIdx.x * p.queue_len + slot) * kInstrWords;
}

__device__ __forceinline__ void stamp(const Params &p, int slot, int event, long long t_start) {
    if (p.flags & MK_STEP_TIMINGS)
        p.timings[((size_t)blockIdx.x * p.queue_len + slot) * kTimingSlots + event] = (int)(clock64() - t_start);
}

// ---------------------------------------------------------------------------
// loader
// ---------------------------------------------------------------------------

struct Ring {
    uint32_t stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
    }
};

// One 16-row x 2048-column weight tile: first byte, row pitch, owning instruction.
struct Tile {
    const uint8_t *src;
    size_t stride_bytes;
    int opcode;
    int slot;
};

// Walks a worker's instruction queue and yields its weight tiles in the order
// the consumers use them.
template <int NCH>
struct TileCursor {
    int slot = -1;
    int op = 0;
    int idx = 0, cnt = 0;   // block position within the instruction
    int sub = 0, nsub = 1;  // tile position within the block
    int first_block = 0;
    const int *ins = nullptr;
    const bf16 *base = nullptr, *base2 = nullptr;
    size_t row_elems = 0;

    __device__ __forceinline__ bool next(const Params &p, Tile &t) {
        while (true) {
            if (idx < cnt) {
                const int block = (op == 5) ? __ldg(ins + 3 + idx) : first_block + idx;
                const bf16 *w = (op == 5 && sub >= NCH) ? base2 : base;
                const int chunk = (op == 6) ? 0 : (sub % NCH);
                t.src = reinterpret_cast<const uint8_t *>(w + (size_t)block * kBlockRows * row_elems + chunk * kChunkCols);
                t.stride_bytes = row_elems * sizeof(bf16);
                t.opcode = op;
                t.slot = slot;
                if (++sub == nsub) { sub = 0; ++idx; }
                return true;
            }
            if (++slot >= p.queue_len) return false;
            ins = instruction_at(p, slot);
            op = __ldg(ins);
            idx = 0; sub = 0; cnt = 0; nsub = NCH;
            const size_t hidden = p.hidden;
            switch (op) {
            case 1: {
                const int layer = __ldg(ins + 1);
                first_block = __ldg(ins + 2); cnt = __ldg(ins + 3) - first_block;
                base = p.qkv_w + (size_t)layer * p.qkv_rows * hidden; row_elems = hidden;
                break;
            }
            case 4: {
                const int layer = __ldg(ins + 1);
                first_block = __ldg(ins + 2); cnt = __ldg(ins + 3) - first_block;
                row_elems = (size_t)p.hq * p.hd;
                base = p.o_w + (size_t)layer * hidden * row_elems;
                break;
            }
            case 5: {
                const int layer = __ldg(ins + 1);
                cnt = __ldg(ins + 2); nsub = 2 * NCH;  // up tiles, then gate tiles
                base = p.up_w + (size_t)layer * p.inter * hidden;
                base2 = p.gate_w + (size_t)layer * p.inter * hidden;
                row_elems = hidden;
                break;
            }
            case 6: {
                const int layer = __ldg(ins + 1);
                first_block = __ldg(ins + 2); cnt = __ldg(ins + 3) - first_block; nsub = 1;
                row_elems = p.inter;
                base = p.down_w + (size_t)layer * hidden * row_elems + (size_t)__ldg(ins + 4) * kChunkCols;
                break;
            }
            case 7:
                first_block = __ldg(ins + 1); cnt = __ldg(ins + 2) - first_block;
                base = p.lm_w; row_elems = hidden;
                break;
            default:
                break;  // attention ops, no-ops and unknown opcodes stream no weights
            }
            if (cnt < 0) cnt = 0;
        }
    }
};

template <int NCH>
__device__ void loader_role(const Params &p, Smem &s, long long t_start) {
    const uint64_t policy = l2_evict_first_policy();
    Ring ring;
    uint32_t live = 0;  // stages whose most recent fill was actually issued
    TileCursor<NCH> tiles;
    Tile t;
    int last_slot = -1;
    while (tiles.next(p, t)) {
        if (t.slot != last_slot) {
            if (last_slot >= 0) stamp(p, last_slot, kEvLastLoad, t_start);
            stamp(p, t.slot, kEvLoaderStart, t_start);
            last_slot = t.slot;
        }
        wait_mbar(p, s, &s.empty[ring.stage], ring.phase ^ 1u, kFailRing, t.opcode, t.slot, (int)ring.stage);
        if (aborted(s)) {
            live &= ~(1u << ring.stage);
        } else {
            live |= 1u << ring.stage;
            mbar_arrive_expect_tx(&s.full[ring.stage], kTileBytes);
            uint8_t *dst = s.stage[ring.stage];
#pragma unroll 4
            for (int r = 0; r < kBlockRows; ++r)
                bulk_load(dst + r * kRowPitch, t.src + r * t.stride_bytes, kRowBytes, &s.full[ring.stage], policy);
        }
        ring.advance();
    }
    if (last_slot >= 0) stamp(p, last_slot, kEvLastLoad, t_start);
    // Never leave the CTA with copies in flight.  In a clean run every fill has
    // been waited for by the consumers; when aborting, wait here (bounded,
    // ignoring the abort flag) for the last fill of every stage.
    if (aborted(s)) {
        for (uint32_t st = 0; st < (uint32_t)kStages; ++st) {
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

struct ConsumerState {
    Ring ring;
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
    if (ctid == 0) wait_counter(p, s, ctr, expected, opcode, slot);
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
}

// 8 consecutive elements of the residual stream starting at `idx`.  `base` is
// the stream as last written in place; with `merge` the down-projection's
// column-slice partial sums of the previous layer are added one slice at a
// time, each add rounded to bf16, which is the order and rounding of the
// reference interpreter's sequential `hidden += partial` updates.
__device__ __forceinline__ void load_hidden8(const Params &p, const bf16 *base, bool merge, int idx, float (&h)[8]) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(base + idx));
    if (!merge) {
        unpack8(raw, h);
        return;
    }
    // slices in groups of four: all loads of a group are issued before its dependent adds
    bool first = true;
    for (int s0 = 0; s0 < p.down_slices; s0 += 4) {
        uint4 parts[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (s0 + j < p.down_slices)
                parts[j] = __ldcg(reinterpret_cast<const uint4 *>(p.down_partials + (size_t)(s0 + j) * p.hidden + idx));
        if (first) { unpack8(raw, h); first = false; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (s0 + j < p.down_slices) {
                float part[8];
                unpack8(parts[j], part);
#pragma unroll
                for (int i = 0; i < 8; ++i) h[i] = round_bf16(h[i] + part[i]);
            }
        }
    }
    if (first) unpack8(raw, h);
}

// Activation operand of the tensor-core matvec.  Consumer warp `cw` owns input
// columns [cw*256, +256) of every 2048-column chunk; within the warp, lane
// (g = lane/4, t = lane%4) holds for j = 0..7 the eight bf16 values of columns
// cw*256 + j*32 + t*8 .. +7 (one uint4).  All eight g-groups hold the same
// values: the MMA's eight output columns are copies and only column 0 is kept.
template <int NCH>
using XOperand = uint4[NCH][8];

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    // both inputs already hold bf16-representable values
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
}

// RMSNorm of the residual stream (reference python_vm.py:50-56): fp32
// statistics; the normalised value is rounded to bf16 and then multiplied by the
// bf16 weight with a second rounding.  Thread `ctid` normalises elements
// [c*2048 + ctid*8, +8) of chunk c; the result goes through shared memory to be
// re-read in the operand layout above.
template <int NCH>
__device__ __forceinline__ void load_normed(const Params &p, Smem &s, int ctid, uint32_t &toggle, const bf16 *base,
                                            bool merge, const bf16 *norm_w, uint4 (&x)[NCH][8]) {
    const int lane = ctid & 31, cw = ctid >> 5;
    uint4 wraw[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) wraw[c] = __ldg(reinterpret_cast<const uint4 *>(norm_w + c * kChunkCols + ctid * 8));
    float h[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        load_hidden8(p, base, merge, c * kChunkCols + ctid * 8, h[c]);
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
        for (int j = 0; j < 8; ++j) x[c][j] = lds128(&s.xbuf[c * kChunkCols + cw * 256 + j * 32 + t * 8]);
}

template <int NCH>
__device__ __forceinline__ void load_plain(const bf16 *vec, int ctid, uint4 (&x)[NCH][8]) {
    const int cw = ctid >> 5, t = ctid & 3;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            x[c][j] = __ldcg(reinterpret_cast<const uint4 *>(vec + c * kChunkCols + cw * 256 + j * 32 + t * 8));
}

// D += A(16x16, bf16) * B(16x8, bf16), fp32 accumulate, on the tensor cores.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    // volatile: keeps the hand-written load/MMA interleaving (two loads in flight per MMA pair)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 16-row block: NCH tiles from the ring times the register-resident
// activation operand.  Lane (g, t) feeds rows g and g+8 of the tile straight
// from shared memory as MMA A-fragments: its 16-byte load at column offset
// j*32 + t*8 supplies the k-slots {2t, 2t+1, 2t+8, 2t+9} of two MMAs, and the
// activation operand uses the same column-to-slot assignment, so no shuffle or
// conversion is needed.  The per-warp results (16 rows) go to the storer.
template <int NCH>
__device__ __forceinline__ void consume_block(const Params &p, Smem &s, ConsumerState &st, int lane, int cw,
                                              const uint4 (&x)[NCH][8], int opcode, int slot) {
    float acc_a[4] = {0.f, 0.f, 0.f, 0.f}, acc_b[4] = {0.f, 0.f, 0.f, 0.f};
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        wait_mbar(p, s, &s.full[st.ring.stage], st.ring.phase, kFailRing, opcode, slot, (int)st.ring.stage);
        const uint8_t *row_g = s.stage[st.ring.stage] + g * kRowPitch + cw * 512 + t * 16;
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
__device__ void attention_partial(const Params &p, Smem &s, int ctid, const int *ins, int slot, long long t_start) {
    constexpr int V = DPL / 8;   // 16-byte vectors per row per lane
    constexpr int kDepth = DPL == 8 ? 4 : 2;  // rows in flight per lane (register budget)
    const int lane = ctid & 31, cw = ctid >> 5;
    const int layer = __ldg(ins + 1), kv_head = __ldg(ins + 2), num_partials = __ldg(ins + 3), part = __ldg(ins + 4);
    const int D = p.hd;
    const int blocks_per_head = D / kBlockRows;

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

    auto load_row = [&](uint4 (&kq)[V], uint4 (&vq)[V], int t) {
#pragma unroll
        for (int v = 0; v < V; ++v) {
            kq[v] = __ldcg(reinterpret_cast<const uint4 *>(kbase + (size_t)t * tok_stride) + v);
            vq[v] = __ldcg(reinterpret_cast<const uint4 *>(vbase + (size_t)t * tok_stride) + v);
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

    if (ctid == 0) {
        stamp(p, slot, kEvAtWait, t_start);
        for (int i = 0; i < kGroup; ++i)
            wait_counter(p, s, counter(p, layer, 0, kv_head * kGroup + i), blocks_per_head, 2, slot);
        wait_counter(p, s, counter(p, layer, 0, p.hq + kv_head), blocks_per_head, 2, slot);
        wait_counter(p, s, counter(p, layer, 0, p.hq + p.hkv + kv_head), blocks_per_head, 2, slot);
        stamp(p, slot, kEvDoneWait, t_start);
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);

    uint4 q[V];
#pragma unroll
    for (int v = 0; v < V; ++v)
        q[v] = __ldcg(reinterpret_cast<const uint4 *>(p.q_post + (size_t)(kv_head * kGroup + h) * D + d0) + v);
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

    const int n_iter = (t1 - t0 + kConsumerWarps - 1) / kConsumerWarps;  // same for every warp
#pragma unroll 1
    for (int base = 0; base < n_iter; base += kDepth) {
#pragma unroll
        for (int j = 0; j < kDepth; ++j) {
            if (base + j < n_iter) {
                const int t = my_first + (base + j) * kConsumerWarps;
                float d = 0.f;
                float vf[DPL];
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    float kf[8];
                    unpack8(kq[j][v], kf);
                    d = dot8(q[v], kf, d);
                    float tmp[8];
                    unpack8(vq[j][v], tmp);
#pragma unroll
                    for (int i = 0; i < 8; ++i) vf[8 * v + i] = tmp[i];
                }
                const int t_next = t + kDepth * kConsumerWarps;
                if (t_next < t1) load_row(kq[j], vq[j], t_next);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                if (t < t1) {
                    const float sc = d * scale_log2e;
                    const float mn = fmaxf(m, sc);
                    const float corr = exp2f(m - mn);  // exp2(-inf) = 0 on the first row
                    const float pr = exp2f(sc - mn);
                    l = l * corr + pr;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pr, vf[i], acc[i] * corr);
                    m = mn;
                }
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

    // merge the 8 warps; one (head, dim) output per thread iteration
    for (int idx = ctid; idx < kGroup * D; idx += kConsumerThreads) {
        const int h = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, s.attn[w][h][kMaxHeadDim]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const float mw = s.attn[w][h][kMaxHeadDim];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            L = fmaf(s.attn[w][h][kMaxHeadDim + 1], f, L);
            O = fmaf(s.attn[w][h][d], f, O);
        }
        const float out = (L > 0.f) ? O / L : 0.f;
        const int head = kv_head * kGroup + h;
        if (!aborted(s)) {
            if (p.skip_attn_reduction) {
                p.attn_out[(size_t)head * D + d] = __float2bfloat16_rn(out);
            } else {
                p.attn_oi[((size_t)head * p.max_partials + part) * D + d] = out;
                // log2 of the natural-exponent sum (reference python_vm.py:323); M is already in log2 units
                if (d == 0)
                    p.attn_lse[(size_t)head * p.max_partials + part] = (L > 0.f) ? M + log2f(L) : -INFINITY;
            }
        }
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);  // all stores issued; s.attn reusable
    if (ctid == 0) stamp(p, slot, 58, t_start);  // outputs stored
    if (ctid == 0 && !aborted(s)) {
        if (p.skip_attn_reduction) {
            red_release_gpu_add(counter(p, layer, 2, 0), kGroup);
        } else {
            fence_acq_rel_gpu();
            for (int h = 0; h < kGroup; ++h) red_relaxed_gpu_add(counter(p, layer, 1, kv_head * kGroup + h), 1);
        }
        stamp(p, slot, kEvOutputReady, t_start);
    }
}

// Log-sum-exp merge of attention partials for 4 heads (reference
// python_vm.py:349-393).  Weights are exp2(lse - max); a non-terminal merge
// stores the natural log of the weight sum as the reference does.
__device__ void attention_reduction(const Params &p, Smem &s, int ctid, const int *ins, int slot, long long t_start) {
    const int layer = __ldg(ins + 1), head0 = __ldg(ins + 2), num_partials = __ldg(ins + 3);
    const int terminal = __ldg(ins + 4), n = __ldg(ins + 5);
    const int out_slot = __ldg(ins + 6 + n);
    const int D = p.hd;
    if (ctid == 0) {
        stamp(p, slot, kEvAtWait, t_start);
        for (int h = 0; h < kGroup; ++h) wait_counter(p, s, counter(p, layer, 1, head0 + h), num_partials, 3, slot);
        stamp(p, slot, kEvDoneWait, t_start);
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    for (int idx = ctid; idx < kGroup * D; idx += kConsumerThreads) {
        const int h = idx / D, d = idx % D;
        const int head = head0 + h;
        const float *lse = p.attn_lse + (size_t)head * p.max_partials;
        const float *oi = p.attn_oi + (size_t)head * p.max_partials * D + d;
        float mx = -INFINITY;
        for (int j = 0; j < n; ++j) mx = fmaxf(mx, __ldcg(lse + __ldg(ins + 6 + j)));
        float denom = 0.f, num = 0.f;
        for (int j = 0; j < n; ++j) {
            const int src = __ldg(ins + 6 + j);
            const float f = exp2f(__ldcg(lse + src) - mx);
            denom += f;
            num = fmaf(__ldcg(oi + (size_t)src * D), f, num);
        }
        const float out = num / denom;
        if (!aborted(s)) {
            if (terminal) {
                p.attn_out[(size_t)head * D + d] = __float2bfloat16_rn(out);
            } else {
                p.attn_oi[((size_t)head * p.max_partials + out_slot) * D + d] = out;
                if (d == 0) p.attn_lse[(size_t)head * p.max_partials + out_slot] = logf(denom);
            }
        }
    }
    named_barrier_sync(kConsumerBarrier, kConsumerThreads);
    if (ctid == 0 && !aborted(s)) {
        red_release_gpu_add(counter(p, layer, 2, 0), kGroup);
        stamp(p, slot, kEvOutputReady, t_start);
    }
}

template <int NCH>
__device__ void consumer_role(const Params &p, Smem &s, int ctid, long long t_start) {
    const int lane = ctid & 31, cw = ctid >> 5;
    ConsumerState st;
    const bf16 *token_row = nullptr;
    if (p.flags & MK_STEP_EMBED) token_row = p.embed_w + (size_t)__ldg(p.token_in) * p.hidden;

#pragma unroll 1
    for (int slot = 0; slot < p.queue_len; ++slot) {
        const int *ins = instruction_at(p, slot);
        const int op = __ldg(ins);
        if (op == 0) continue;
        if (ctid == 0) stamp(p, slot, kEvConsumerStart, t_start);
        uint4 x[NCH][8];
        switch (op) {
        case 1: {
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3);
            if (layer > 0) {
                if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
                consumer_wait(p, s, ctid, counter(p, layer - 1, 5, 0), p.down_total, op, slot);
                if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            }
            const bf16 *base = (layer == 0 && token_row) ? token_row : p.hidden_states;
            load_normed<NCH>(p, s, ctid, st.norm_toggle, base, layer > 0, p.attn_norm_w + (size_t)layer * p.hidden, x);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH>(p, s, st, lane, cw, x, op, slot);
            break;
        }
        case 2:
            if (p.hd == 64) attention_partial<8>(p, s, ctid, ins, slot, t_start);
            else attention_partial<16>(p, s, ctid, ins, slot, t_start);
            break;
        case 3:
            attention_reduction(p, s, ctid, ins, slot, t_start);
            break;
        case 4: {
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3);
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, layer, 2, 0), p.hq, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_plain<NCH>(p.attn_out, ctid, x);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH>(p, s, st, lane, cw, x, op, slot);
            break;
        }
        case 5: {
            const int layer = __ldg(ins + 1), n = __ldg(ins + 2);
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, layer, 3, 0), p.hidden / kBlockRows, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_normed<NCH>(p, s, ctid, st.norm_toggle, p.hidden_states, false, p.mlp_norm_w + (size_t)layer * p.hidden, x);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int i = 0; i < n; ++i) {
                consume_block<NCH>(p, s, st, lane, cw, x, op, slot);  // up rows
                consume_block<NCH>(p, s, st, lane, cw, x, op, slot);  // gate rows
            }
            break;
        }
        case 6: {
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3), red = __ldg(ins + 4);
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            // only the gate/up rows of this 2048-column slice have to be ready
            consumer_wait(p, s, ctid, counter(p, layer, kSliceCounterRow, red), kChunkCols / kBlockRows, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            uint4 xs[1][8];
            load_plain<1>(p.silu_out + (size_t)red * kChunkCols, ctid, xs);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<1>(p, s, st, lane, cw, xs, op, slot);
            break;
        }
        case 7: {
            const int b0 = __ldg(ins + 1), b1 = __ldg(ins + 2);
            if (ctid == 0) stamp(p, slot, kEvAtWait, t_start);
            consumer_wait(p, s, ctid, counter(p, p.layers - 1, 5, 0), p.down_total, op, slot);
            if (ctid == 0) stamp(p, slot, kEvDoneWait, t_start);
            load_normed<NCH>(p, s, ctid, st.norm_toggle, p.hidden_states, true, p.lm_norm_w, x);
            if (ctid == 0) stamp(p, slot, kEvFirstUse, t_start);
            for (int b = b0; b < b1; ++b) consume_block<NCH>(p, s, st, lane, cw, x, op, slot);
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

__device__ __forceinline__ void publish(const Params &p, Smem &s, int lane, int *ctr, int value) {
    __syncwarp();
    if (lane == 0 && !aborted(s)) red_release_gpu_add(ctr, value);
}

__device__ __forceinline__ unsigned long long argmax_key(float logit_bf16, int index) {
    // Order-preserving map of the bf16 bit pattern; ties resolve to the lowest index.
    uint32_t bits = __float_as_uint(logit_bf16) >> 16;
    bits = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
    return ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (uint32_t)index);
}

template <int NCH>
__device__ void storer_role(const Params &p, Smem &s, int lane, long long t_start) {
    StorerState st;
    const int D = p.hd;
    const int k_start = p.hq * D, v_start = k_start + p.hkv * D;
    const bf16 *token_row = nullptr;
    if (p.flags & MK_STEP_EMBED) token_row = p.embed_w + (size_t)__ldg(p.token_in) * p.hidden;

#pragma unroll 1
    for (int slot = 0; slot < p.queue_len; ++slot) {
        const int *ins = instruction_at(p, slot);
        const int op = __ldg(ins);
        if (op == 0) continue;
        if (lane == 0) stamp(p, slot, kEvStorerStart, t_start);
        switch (op) {
        case 1: {
            // bf16(matvec) -> RoPE in fp32 on Q and K rows -> bf16 store
            // (reference python_vm.py:196-248, llama.py:136-174)
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3);
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
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot));
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
                if (lane < kBlockRows && !aborted(s)) {
                    const bf16 o = __float2bfloat16_rn(out);
                    if (row < k_start) p.q_post[row] = o;
                    else if (row < v_start) p.k_cache[cache_row + (row - k_start)] = o;
                    else p.v_cache[cache_row + (row - v_start)] = o;
                }
            }
            // one counter per head; the first release also covers the later heads' rows
            const int bph = D / kBlockRows;
            __syncwarp();
            if (lane == 0) stamp(p, slot, 59, t_start);  // outputs issued, before the fence
            if (lane == 0 && !aborted(s)) {
                fence_acq_rel_gpu();  // once; the adds below are relaxed
                for (int head = b0 / bph; head <= (b1 - 1) / bph; ++head) {
                    const int lo = max(b0, head * bph), hi = min(b1, (head + 1) * bph);
                    red_relaxed_gpu_add(counter(p, layer, 0, head), hi - lo);
                }
            }
            break;
        }
        case 4: {
            // hidden[rows] = bf16(hidden[rows] + bf16(matvec)) (reference python_vm.py:59-104)
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3);
            const bf16 *base = (layer == 0 && token_row) ? token_row : p.hidden_states;
            auto residual = [&](int row) {
                float h = ldcg_bf16(base + row);
                if (layer > 0)
                    for (int sl = 0; sl < p.down_slices; ++sl)
                        h = round_bf16(h + ldcg_bf16(p.down_partials + (size_t)sl * p.hidden + row));
                return h;
            };
            // The residual rows were finished by the previous layer.  If its last
            // counter already shows that, fetch the first block's rows now instead
            // of after the sums arrive (this warp is idle until then).
            const bool early = layer == 0 || ld_acquire_gpu(counter(p, layer - 1, 5, 0)) >= p.down_total;
            float h_first = 0.f;
            if (early && lane < kBlockRows) h_first = residual(b0 * kBlockRows + lane);
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot));
                if (lane < kBlockRows && !aborted(s)) {
                    const int row = b * kBlockRows + lane;
                    const float h = (early && b == b0) ? h_first : residual(row);
                    p.hidden_states[row] = __float2bfloat16_rn(h + y);
                }
            }
            publish(p, s, lane, counter(p, layer, 3, 0), b1 - b0);
            break;
        }
        case 5: {
            // bf16(bf16(silu(bf16 gate)) * bf16 up) (reference python_vm.py:146-165)
            const int layer = __ldg(ins + 1), n = __ldg(ins + 2);
            for (int i = 0; i < n; ++i) {
                const int b = __ldg(ins + 3 + i);
                const float up = round_bf16(collect_block(p, s, st, lane, op, slot));
                const float gate = round_bf16(collect_block(p, s, st, lane, op, slot));
                if (lane < kBlockRows && !aborted(s)) {
                    const float act = round_bf16(gate / (1.0f + expf(-gate)));
                    p.silu_out[b * kBlockRows + lane] = __float2bfloat16_rn(act * up);
                }
            }
            // per 2048-column slice of silu_out (what one down-projection
            // instruction reads), then the reference interpreter's single counter
            const int my_slice = lane < n ? (__ldg(ins + 3 + lane) * kBlockRows) / kChunkCols : -1;
            __syncwarp();
            if (lane == 0) stamp(p, slot, 59, t_start);  // outputs issued, before the fence
            if (lane == 0) fence_acq_rel_gpu();  // once; the adds below are relaxed
            for (int sl = 0; sl < p.down_slices; ++sl) {
                const int cnt = __popc(__ballot_sync(0xffffffffu, my_slice == sl));
                if (lane == 0 && cnt && !aborted(s)) red_relaxed_gpu_add(counter(p, layer, kSliceCounterRow, sl), cnt);
            }
            if (lane == 0 && !aborted(s)) red_relaxed_gpu_add(counter(p, layer, 4, 0), n);
            break;
        }
        case 6: {
            // bf16(matvec over one 2048-column slice), parked per slice; the
            // consumers of the residual stream add the slices in slice order.
            const int layer = __ldg(ins + 1), b0 = __ldg(ins + 2), b1 = __ldg(ins + 3), red = __ldg(ins + 4);
            for (int b = b0; b < b1; ++b) {
                const float y = collect_block(p, s, st, lane, op, slot);
                if (lane < kBlockRows && !aborted(s))
                    p.down_partials[(size_t)red * p.hidden + b * kBlockRows + lane] = __float2bfloat16_rn(y);
            }
            publish(p, s, lane, counter(p, layer, 5, 0), b1 - b0);
            break;
        }
        case 7: {
            const int b0 = __ldg(ins + 1), b1 = __ldg(ins + 2);
            unsigned long long best = 0ull;
            for (int b = b0; b < b1; ++b) {
                const float y = round_bf16(collect_block(p, s, st, lane, op, slot));
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

template <int NCH>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long t_start = clock64();

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kConsumerWarps);
        }
        for (int i = 0; i < kPartialBufs; ++i) {
            mbar_init(&s.pfull[i], kConsumerWarps);
            mbar_init(&s.pempty[i], 1);
        }
        s.abort_flag = 0;
        s.is_last = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) loader_role<NCH>(p, s, t_start);
        __syncwarp();
    } else if (warp < kStorerWarp) {
        consumer_role<NCH>(p, s, tid - 32, t_start);
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

    // Residual stream: fold in the last down-projection's slice sums unless an
    // o_proj of the following layer already did.
    int pending_layer = -1;
    for (int l = p.layers - 1; l >= 0; --l) {
        if (ld_acquire_gpu(counter(p, l, 5, 0)) != 0) { pending_layer = l; break; }
    }
    if (pending_layer >= 0 && ld_acquire_gpu(counter(p, pending_layer, 5, 0)) >= p.down_total &&
        (pending_layer == p.layers - 1 || ld_acquire_gpu(counter(p, pending_layer + 1, 3, 0)) == 0)) {
        for (int idx = tid; idx < p.hidden; idx += kThreads) {
            float h = ldcg_bf16(p.hidden_states + idx);
            for (int sl = 0; sl < p.down_slices; ++sl)
                h = round_bf16(h + ldcg_bf16(p.down_partials + (size_t)sl * p.hidden + idx));
            p.hidden_states[idx] = __float2bfloat16_rn(h);
        }
    }
    if (tid == 0) {
        const unsigned long long key = __ldcg(p.argmax_key);
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

struct Handle {
    MkModelDesc desc;
    Params params;
    int device = 0;
    int nch = 1;
    int sm_count = 0;
    int resident = 0;
    cudaFuncAttributes attrs;
    size_t smem_bytes = 0;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
};

static const void *kernel_for(int nch) {
    return nch == 2 ? reinterpret_cast<const void *>(&decode_step_kernel<2>)
                    : reinterpret_cast<const void *>(&decode_step_kernel<1>);
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
    if (d->weight_format != MK_WEIGHTS_BF16)
        return fail(MK_ERR_UNSUPPORTED, "mk_create: weight format %d not supported by this build", d->weight_format);
    const int H = d->hidden_size, D = d->head_dim;
    if (H <= 0 || d->num_layers <= 0 || d->num_q_heads <= 0 || d->num_kv_heads <= 0 || D <= 0 ||
        d->intermediate_size <= 0 || d->vocab_size <= 0)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_create: non-positive dimension");
    if (H != kChunkCols && H != 2 * kChunkCols)
        return fail(MK_ERR_UNSUPPORTED, "hidden_size %d: kernel streams 2048-column tiles, hidden must be 2048 or 4096", H);
    if (d->num_q_heads * D != H) return fail(MK_ERR_UNSUPPORTED, "num_q_heads*head_dim (%d) must equal hidden_size (%d)", d->num_q_heads * D, H);
    if (D != 64 && D != 128) return fail(MK_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", D);
    if (d->num_q_heads != kGroup * d->num_kv_heads)
        return fail(MK_ERR_UNSUPPORTED, "query group size must be %d (got %d q heads, %d kv heads)", kGroup, d->num_q_heads, d->num_kv_heads);
    if (d->intermediate_size % kChunkCols) return fail(MK_ERR_UNSUPPORTED, "intermediate_size %d not a multiple of 2048", d->intermediate_size);
    if (d->vocab_size % kBlockRows) return fail(MK_ERR_UNSUPPORTED, "vocab_size %d not a multiple of 16", d->vocab_size);
    if (d->barrier_rows < 8 || d->barrier_cols < d->num_q_heads + 2 * d->num_kv_heads)
        return fail(MK_ERR_BAD_ARGUMENT, "barriers tensor too small: rows %d cols %d", d->barrier_rows, d->barrier_cols);
    if (d->kv_batch < 1 || d->kv_max_len < 1 || d->rope_positions < 1 || d->max_partials < 1)
        return fail(MK_ERR_BAD_ARGUMENT, "mk_create: cache/rope/partials extent must be positive");
    const void *required[] = {d->qkv_w, d->o_w, d->up_w, d->gate_w, d->down_w, d->lm_head_w, d->attn_norm_w,
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
    cudaError_t e = cudaGetDevice(&h->device);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaGetDevice"); }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, h->device);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaGetDeviceProperties"); }
    h->sm_count = prop.multiProcessorCount;
    if (!prop.cooperativeLaunch) { delete h; return fail(MK_ERR_RESIDENCY, "device does not support cooperative launch"); }

    const void *kern = kernel_for(h->nch);
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

    // scratch: [down_slices][hidden] bf16 | argmax key (8 B) | done counter | status[8]
    const int slices = d->intermediate_size / kChunkCols;
    const size_t partial_bytes = ((size_t)slices * H * sizeof(bf16) + 255) & ~size_t(255);
    h->scratch_bytes = partial_bytes + 256;
    e = cudaMalloc(&h->scratch, h->scratch_bytes);
    if (e != cudaSuccess) { delete h; return cuda_fail(e, "cudaMalloc(scratch)"); }
    e = cudaMemset(h->scratch, 0, h->scratch_bytes);
    if (e != cudaSuccess) { cudaFree(h->scratch); delete h; return cuda_fail(e, "cudaMemset(scratch)"); }

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
    p.down_partials = (bf16 *)sc;
    p.argmax_key = (unsigned long long *)(sc + partial_bytes);
    p.done_counter = (int *)(sc + partial_bytes + 16);
    p.status = (int *)(sc + partial_bytes + 32);
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
    cudaError_t e = cudaLaunchCooperativeKernel(kernel_for(h->nch), dim3(p.workers), dim3(kThreads), args,
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
    info->stage_count = kStages;
    info->stage_bytes = kStageBytes;
    info->resident_ctas_per_sm = h->resident;
    info->queue_len = h->params.queue_len;
    info->scratch_bytes = (int64_t)h->scratch_bytes;
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
        cudaMemset(h->params.argmax_key, 0, 256);
        return fail(MK_ERR_DEVICE_WAIT, "device wait expired: code %d worker %d opcode %d slot %d saw %d expected %d",
                    words[0], words[1], words[2], words[3], words[4], words[5]);
    }
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
    default:
        return fail(MK_ERR_BAD_ARGUMENT, "mk_set_option: unknown option %d", option);
    }
}

extern "C" void mk_destroy(void *handle) {
    Handle *h = (Handle *)handle;
    if (!h) return;
    cudaFree(h->scratch);
    delete h;
}
