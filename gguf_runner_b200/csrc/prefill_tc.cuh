// Flash-style causal / windowed GQA prefill on the 5th-generation tensor cores.
//
// Device counterpart of the per-token prefill loop of the reference
// (src/engine/runtime/inference.rs:2981-3017 calling attention_token :1970):
// every query row sees exactly the key interval visible_keys gives it
// (src/engine/runtime/attention.rs:73-97). RoPE and the cache append have
// already been applied by rope_append_kernel; K and V tiles are read from the
// bf16 cache rows themselves.
//
// A work item is two consecutive 128-row query tiles of one query head; its CTA
// walks the visible 128-key tiles of the KV head. The kernel is persistent: one
// CTA per SM takes items, longest first, from a device-wide counter, and the
// producer runs ahead into the next item, so that the load latency and most of
// the pipeline ramp of an item hide behind the tail of the previous one.
//   warp 8       scheduler + TMA producer: Q tiles of the item, then K and V tiles
//                into 2-stage rings (cp.async.bulk.tensor, 128-byte swizzle,
//                mbarrier complete_tx)
//   warp 9       MMA issuer: S_t = Q_t K^T and O_t += P_t V with tcgen05.mma,
//                accumulators in TMEM (S0 S1 O0 O1 = 512 columns); P_t is read
//                straight from TMEM where the softmax wrote it over S_t, in two
//                64-key halves so that P V starts before the softmax has finished
//                the tile
//   warps 0-3    softmax of query tile 0 (one thread per query row)
//   warps 4-7    softmax of query tile 1
// The two query tiles ping-pong: while one tile's softmax runs on the CUDA
// cores, the tensor core works on the other tile. Online softmax with base-2
// exponentials; O is rescaled in TMEM only when a row maximum grows by more
// than 2^8 (the stale maximum stays exact because l uses the same reference).
//
// Every wait is bounded: when a limit runs out the CTA raises an abort flag,
// all roles leave their loops, TMEM is freed and the host sees GGR_ERR_TIMEOUT.
#pragma once

#include <string>

#include "common.cuh"
#include "sm100_utils.cuh"

namespace ggr {

struct PrefillTcArgs {
    KvView kv;
    Visibility vis;
    int layer, seq, base_pos, m;
    const __nv_bfloat16* q;  // [m][Hq*D] rotated queries (bf16)
    float* out;              // [m][Hq*D]
    float score_scale;       // (1/sqrt(D) or 1) * log2(e)
    int* err;                // device-visible error word (mapped host memory)
    int* sched;              // [0] work items handed out beyond the first wave, [1] CTAs that have left (persistent kernel)
    int n_items;             // query-tile pairs x query heads
    // optional output gate (src/engine/runtime/inference.rs:3509-3519), f32 or bf16: head h of row i at
    // gate + (i * Hq + h) * gate_head_stride elements
    const void* gate;
    int gate_bf16, gate_head_stride;
    // launched with programmatic stream serialisation behind the rope / append kernel of the same call: the CTA sets
    // itself up (barriers, tensor memory) while that kernel drains and waits for it before it touches memory
    int dependent;
#ifdef GGR_TC_TRACE
    long long* trace;        // cycle counters of CTA 0 (diagnostic builds only)
#endif
};

// cycle-trace hooks of diagnostic builds (-DGGR_TC_TRACE); empty otherwise
#ifdef GGR_TC_TRACE
#define TRACE_ADD(var) do { long long now_ = clock64(); var += now_ - tr_x; tr_x = now_; } while (0)
#define TRACE_MARK() tr_x = clock64()
// absolute time stamps of four mid-kernel steps: slot layout [step - 16][24]
#define TRACE_EVT(step, slot) do { if (blockIdx.x == 0 && it == 0 && a.trace && (threadIdx.x & 31) == 0 && (step) >= 16 && (step) < 20) \
        a.trace[32 + ((step) - 16) * 24 + (slot)] = clock64(); } while (0)
#else
#define TRACE_EVT(step, slot)
#define TRACE_ADD(var)
#define TRACE_MARK()
#endif

// out = finite_or_zero(o * sigmoid(gate)) on four consecutive head elements (src/engine/kernels/math.rs:399-402)
__device__ __forceinline__ float4 prefill_gate4(float4 o, const void* gate_row, int gate_bf16, int d) {
    float g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        g[i] = gate_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(gate_row)[d + i])
                         : static_cast<const float*>(gate_row)[d + i];
    float r[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float v = r[i] * (1.0f / (1.0f + expf(-g[i])));
        r[i] = isfinite(v) ? v : 0.0f;
    }
    return make_float4(r[0], r[1], r[2], r[3]);
}

constexpr int kTcBM = 128;       // query rows per tile
constexpr int kTcBN = 128;       // keys per tile
constexpr int kTcThreads = 384;  // 8 softmax warps + a control warpgroup (producer, MMA issuer, 2 idle)
// Which of every four 4-score groups compute their second score pair with ex2_poly_x2 instead of the MUFU
// unit: bit g set = group g. 0x5 moves a quarter of all exponentials to the FMA pipe.
#ifndef GGR_EXP_POLY_MASK
#define GGR_EXP_POLY_MASK 0x5
#endif
constexpr int kExpPolyMask = GGR_EXP_POLY_MASK;
// registers per thread after the split: control warpgroup (producer, MMA issuer) / softmax warpgroups
#ifndef GGR_TC_CTRL_REGS
#define GGR_TC_CTRL_REGS 88
#define GGR_TC_SOFTMAX_REGS 208
#endif
constexpr int kTcCtrlRegs = GGR_TC_CTRL_REGS, kTcSoftmaxRegs = GGR_TC_SOFTMAX_REGS;
static_assert(tc::RegSplitOk<kTcCtrlRegs, kTcSoftmaxRegs>::value, "setmaxnreg split would never complete");


// Geometry of one work item: two consecutive 128-row query tiles of one query head.
struct TcItem {
    int h, kvh, q_row0;
    int lo0, hi0, lo1, hi1;  // visible 128-key tiles [lo_t, hi_t) of query tile t (ranges are monotone in the position)
    int lo, hi;              // their union: the key tiles the CTA walks
    __device__ __forceinline__ int lo_of(int t) const { return t ? lo1 : lo0; }
    __device__ __forceinline__ int hi_of(int t) const { return t ? hi1 : hi0; }
    __device__ __forceinline__ bool active(int t, int j) const { return j >= lo_of(t) && j < hi_of(t); }
};

// Items are numbered longest first: late query rows see the most keys.
__device__ __forceinline__ TcItem tc_item(const PrefillTcArgs& a, int r) {
    TcItem it;
    const int Hq = a.kv.Hq;
    const int n_pairs = (a.m + 2 * kTcBM - 1) / (2 * kTcBM);
    const int pair = n_pairs - 1 - r / Hq;
    it.h = r % Hq;
    it.kvh = it.h / a.kv.G;
    it.q_row0 = pair * 2 * kTcBM;
    int lo_t[2], hi_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int r0 = it.q_row0 + t * kTcBM;
        if (r0 >= a.m) {
            lo_t[t] = hi_t[t] = 0;
            continue;
        }
        const int r1 = min(a.m, r0 + kTcBM) - 1;
        int vs0, ve0, vs1, ve1;
        a.vis.range(a.base_pos + r0, vs0, ve0);
        a.vis.range(a.base_pos + r1, vs1, ve1);
        lo_t[t] = min(vs0, vs1) / kTcBN;
        hi_t[t] = (max(ve0, ve1) + kTcBN - 1) / kTcBN;
    }
    it.lo0 = lo_t[0], it.hi0 = hi_t[0], it.lo1 = lo_t[1], it.hi1 = hi_t[1];
    const bool act0 = it.hi0 > it.lo0, act1 = it.hi1 > it.lo1;
    it.lo = act0 ? it.lo0 : it.lo1;
    it.hi = act0 ? it.hi0 : it.hi1;
    if (act0 && act1) {
        it.lo = min(it.lo0, it.lo1);
        it.hi = max(it.hi0, it.hi1);
    }
    return it;
}

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, PrefillTcArgs a) {
    using namespace tc;
    constexpr int NBLK = D / 64;                    // 64-element (128-byte) column blocks of a tile
    constexpr uint32_t BLK_BYTES = 128 * 128;       // one [128 rows][128 bytes] swizzled block
    constexpr uint32_t TILE_BYTES = NBLK * BLK_BYTES;
    constexpr uint32_t O_COL0 = 256;                // S0 at 0, S1 at 128, O tiles from 256

    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[24];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_item[2];

    // the warp index goes through a broadcast so that the compiler knows the role branches are warp-uniform
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base;                       // [2][TILE_BYTES]
    const uint32_t sK = sQ + 2 * TILE_BYTES;             // [2 stages][TILE_BYTES]
    const uint32_t sV = sK + 2 * TILE_BYTES;             // [2 stages][TILE_BYTES]
    const uint32_t sOut = sV + 2 * TILE_BYTES;           // [8 softmax warps][32 rows][128 bytes]: output staging

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8u;
    auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (4 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (6 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (8 + s); };
    auto s_full = [&](int t) { return bar0 + 8u * (10 + t); };
    auto p_half = [&](int t, int half) { return bar0 + 8u * (12 + 2 * t + half); };  // P_t keys 0-63 / 64-127 stored
    auto o_final = [&](int t) { return bar0 + 8u * (16 + t); };   // all P V of the item have landed in O_t
    auto o_free = [&](int t) { return bar0 + 8u * (18 + t); };    // the softmax warps have read O_t out
    auto item_full = [&](int s) { return bar0 + 8u * (20 + s); };
    auto item_empty = [&](int s) { return bar0 + 8u * (22 + s); };

    if (tid == 0) {
        s_abort = 0;
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1);
            mbar_init(p_half(s, 0), kTcBM);
            mbar_init(p_half(s, 1), kTcBM);
            mbar_init(o_final(s), 1);
            mbar_init(o_free(s), kTcBM);
            mbar_init(item_full(s), 1);
            mbar_init(item_empty(s), 9);  // lane 0 of the eight softmax warps and of the MMA issuer
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(&s_tmem_base), 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = s_tmem_base;
    volatile int* abortp = &s_abort;
    volatile int* itemp = s_item;
    const int64_t row_base = a.kv.row(a.seq, a.layer, 0);
    const int Hq = a.kv.Hq;
    if (a.dependent) asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp >= 8) {
      // control warpgroup: gives registers up; warps 10 and 11 have no role
      reg_release<kTcCtrlRegs>();
      if (warp == 8) {
        // ---------------- scheduler + TMA producer ----------------
        // Fetches the CTA's next work item (the first one is its block index, later ones come from a
        // device-wide counter), publishes it to the other roles and runs ahead of them: Q of the next item is
        // requested as soon as the last Q K^T of the current one has completed, K and V tiles as stages free up.
        if (lane == 0) {
            int g = 0;  // K / V tiles requested so far (ring position)
            for (int it = 0;; ++it) {
                const int slot = it & 1;
                if (!mbar_wait(item_empty(slot), ((it >> 1) & 1) ^ 1, abortp)) break;
                int r = it == 0 ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(a.sched, 1);
                if (r >= a.n_items) r = -1;
                itemp[slot] = r;
                mbar_arrive(item_full(slot));
                if (r < 0) break;
                const TcItem w = tc_item(a, r);
                const bool act0 = w.hi0 > w.lo0, act1 = w.hi1 > w.lo1;
                if (!mbar_wait(q_empty, (it & 1) ^ 1, abortp)) break;
                mbar_expect_tx(q_full, ((act0 ? 1 : 0) + (act1 ? 1 : 0)) * TILE_BYTES);
                for (int t = 0; t < 2; ++t) {
                    if (!(t == 0 ? act0 : act1)) continue;
                    for (int b = 0; b < NBLK; ++b)
                        tma_load_2d(sQ + t * TILE_BYTES + b * BLK_BYTES, &tmQ, w.h * D + b * 64, w.q_row0 + t * kTcBM, q_full);
                }
                bool ok = true;
                for (int j = w.lo; j < w.hi; ++j, ++g) {
                    const int s = g & 1;
                    const uint32_t ph = ((g >> 1) & 1) ^ 1;
                    const int y = (int)(row_base + (int64_t)j * kTcBN);
                    if (!(ok = mbar_wait(k_empty(s), ph, abortp))) break;
                    mbar_expect_tx(k_full(s), TILE_BYTES);
                    for (int b = 0; b < NBLK; ++b)
                        tma_load_2d(sK + s * TILE_BYTES + b * BLK_BYTES, &tmK, w.kvh * D + b * 64, y, k_full(s));
                    if (!(ok = mbar_wait(v_empty(s), ph, abortp))) break;
                    mbar_expect_tx(v_full(s), TILE_BYTES);
                    for (int b = 0; b < NBLK; ++b)
                        tma_load_2d(sV + s * TILE_BYTES + b * BLK_BYTES, &tmV, w.kvh * D + b * 64, y, v_full(s));
                }
                if (!ok) break;
            }
        }
      } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        // One issuer serves both query tiles in turn. That order is what keeps the tiles in anti-phase (one
        // tile's softmax runs while the tensor core works for the other tile): with one issuer warp per tile
        // both tiles fell into step on the shared K / V stages, their softmaxes competed for the MUFU unit
        // and the kernel was slower. The whole warp runs the loop, one elected lane issues.
        constexpr uint32_t IDESC_QK = idesc_bf16(kTcBN, 0);
        constexpr uint32_t IDESC_PV = idesc_bf16(D, 1);
        // Descriptors are built once; an MMA adds its byte offset (in 16-byte units) to the start
        // address field, so the issue loop is a few integer adds per instruction. (Rebuilding the
        // 64-bit descriptors per MMA under the register cap made every issue cost ~110 cycles.)
        const uint64_t dQ = smem_desc(sQ, 16, 1024), dK = smem_desc(sK, 16, 1024);
        const uint64_t dV = smem_desc(sV, BLK_BYTES, 1024);
        const uint32_t tmem = __shfl_sync(0xffffffffu, s_tmem_base, 0);  // shadows the CTA-wide copy: provably uniform
        auto issue_qk = [&](int t, int s) {
            // S_t = Q_t K^T: both operands K-major, 16 head elements per instruction
            const uint64_t a0 = dQ + (uint64_t)((t * TILE_BYTES) >> 4), b0 = dK + (uint64_t)((s * TILE_BYTES) >> 4);
            const uint32_t d = tmem + t * 128;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t off = ((ks >> 2) * BLK_BYTES + (ks & 3) * 32) >> 4;
                mma_ss_e(d, a0 + off, b0 + off, IDESC_QK, ks > 0 ? 1u : 0u);
            }
        };
        auto issue_pv_half = [&](int t, int s, int half, bool accumulate) {
            // O_t += P_t V over 64 keys: P from TMEM (two bf16 per column), V MN-major, 16 keys per instruction
            const uint64_t b0 = dV + (uint64_t)((s * TILE_BYTES) >> 4);
            const uint32_t d = tmem + O_COL0 + t * D, p0 = tmem + t * 128;
#pragma unroll
            for (int kk = 0; kk < kTcBN / 32; ++kk) {
                const int ks = half * (kTcBN / 32) + kk;
                mma_ts_e(d, p0 + ks * 8, b0 + (uint64_t)((ks * 16 * 128) >> 4), IDESC_PV, (accumulate || ks > 0) ? 1u : 0u);
            }
        };
#ifdef GGR_TC_TRACE
        long long tr_v = 0, tr_p0 = 0, tr_p1 = 0, tr_k = 0, tr_issue = 0, tr_issue_qk = 0, tr_t0 = clock64(), tr_x;
        int tr_steps = 0;
#endif
        int g = 0;             // K / V tiles consumed so far (ring position)
        int c0 = 0, c1 = 0;    // key tiles each query tile has been through (phase of s_full / p_half)
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int slot = it & 1;
            if (!(ok = mbar_wait_warp(item_full(slot), (it >> 1) & 1, abortp))) break;
            // the broadcast tells the compiler that the item is warp-uniform: the tile bounds, ring positions and
            // descriptors derived from it then stay in uniform registers, where tcgen05.mma wants its operands
            const int r = __shfl_sync(0xffffffffu, itemp[slot], 0);
            if (lane == 0) mbar_arrive(item_empty(slot));
            if (r < 0) break;
            const TcItem w = tc_item(a, r);
            const int lo = w.lo, hi = w.hi;
            // Every item moves o_free and o_final of both tiles on by one phase. A tile without visible keys
            // does that here; an active tile waits for o_free right before its first P V overwrites O_t.
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (w.hi_of(t) <= w.lo_of(t)) {
                    if (!(ok = mbar_wait_warp(o_free(t), (it & 1) ^ 1, abortp))) break;
                    if (lane == 0) mbar_arrive(o_final(t));
                }
            if (!ok) break;
            if (!(ok = mbar_wait_warp(q_full, it & 1, abortp))) break;
            if (hi == lo) {
                mma_commit_e(q_empty);
                continue;
            }
            if (!(ok = mbar_wait_warp(k_full(g & 1), (g >> 1) & 1, abortp))) break;
            fence_after_sync();
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (w.active(t, lo)) {
                    issue_qk(t, g & 1);
                    mma_commit_e(s_full(t));
                }
            mma_commit_e(k_empty(g & 1));
            if (hi - lo == 1) mma_commit_e(q_empty);
            for (int j = lo; j < hi; ++j, ++g) {
                const int s = g & 1;
                const bool has_next = j + 1 < hi;
                TRACE_MARK();
                if (!(ok = mbar_wait_warp(v_full(s), (g >> 1) & 1, abortp))) break;
                TRACE_ADD(tr_v);
                TRACE_EVT(j - lo, 6);
                bool next_k_ready = false;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int lo_t = w.lo_of(t), hi_t = w.hi_of(t), c_t = t ? c1 : c0;
                    if (j >= lo_t && j < hi_t) {
                        const uint32_t ph = (c_t + j - lo_t) & 1;
                        if (!(ok = mbar_wait_warp(p_half(t, 0), ph, abortp))) break;
                        if (t == 0) { TRACE_ADD(tr_p0); } else { TRACE_ADD(tr_p1); }
                        TRACE_EVT(j - lo, t * 3);
                        // the previous item's outputs must have left O_t before the first P V overwrites it
                        if (j == lo_t && !(ok = mbar_wait_warp(o_free(t), (it & 1) ^ 1, abortp))) break;
                        fence_after_sync();
                        issue_pv_half(t, s, 0, j > lo_t);
                        if (!(ok = mbar_wait_warp(p_half(t, 1), ph, abortp))) break;
                        fence_after_sync();
                        issue_pv_half(t, s, 1, true);
                        if (j == hi_t - 1) mma_commit_e(o_final(t));
                        TRACE_ADD(tr_issue);
                        TRACE_EVT(j - lo, t * 3 + 1);
                    }
                    if (has_next && j + 1 >= lo_t && j + 1 < hi_t) {
                        if (!next_k_ready) {
                            if (!(ok = mbar_wait_warp(k_full(s ^ 1), ((g + 1) >> 1) & 1, abortp))) break;
                            TRACE_ADD(tr_k);
                            fence_after_sync();
                            next_k_ready = true;
                        }
                        issue_qk(t, s ^ 1);
                        mma_commit_e(s_full(t));
                        TRACE_ADD(tr_issue_qk);
                        TRACE_EVT(j - lo, t * 3 + 2);
                    }
                }
                if (!ok) break;
                mma_commit_e(v_empty(s));
                if (has_next) {
                    mma_commit_e(k_empty(s ^ 1));
                    if (j + 2 == hi) mma_commit_e(q_empty);  // the item's last Q K^T are in flight
                }
            }
            c0 += w.hi0 - w.lo0;
            c1 += w.hi1 - w.lo1;
#ifdef GGR_TC_TRACE
            tr_steps += hi - lo;
#endif
        }
#ifdef GGR_TC_TRACE
        if (blockIdx.x == 0 && a.trace) {
            a.trace[0] = clock64() - tr_t0; a.trace[1] = tr_v; a.trace[2] = tr_p0; a.trace[3] = tr_p1;
            a.trace[4] = tr_k; a.trace[5] = tr_issue; a.trace[6] = tr_steps; a.trace[7] = tr_issue_qk;
        }
#endif
      }
    } else {
        // ---------------- softmax warps: one thread per query row ----------------
        reg_acquire<kTcSoftmaxRegs>();
        const int t = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_addr + t * 128;
        const uint32_t tO = tmem + lane_addr + O_COL0 + t * D;
        const float c = a.score_scale;
        const float thr = 8.0f / c;
        bool ok = true;
        int cs = 0;  // key tiles this query tile has been through (phase of s_full)
#ifdef GGR_TC_TRACE
        long long ts_wait = 0, ts_ld = 0, ts_max = 0, ts_resc = 0, ts_exp = 0, ts_t0 = clock64(), tr_x;
        long long ts_item = 0, ts_ofin = 0, ts_epi = 0, ts_items = 0;
#endif
        for (int it = 0; ok; ++it) {
            const int slot = it & 1;
            TRACE_MARK();
            if (!(ok = mbar_wait(item_full(slot), (it >> 1) & 1, abortp))) break;
            TRACE_ADD(ts_item);
            const int r = itemp[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(item_empty(slot));
            if (r < 0) break;
            const TcItem w = tc_item(a, r);
            const int lo_t = w.lo_of(t), hi_t = w.hi_of(t), n_t = hi_t - lo_t;
#ifdef GGR_TC_TRACE
            const int lo = w.lo;
#endif
            const int qi = w.q_row0 + t * kTcBM + row;
            const bool valid = qi < a.m;
            int vs = 0, ve = 0;
            if (valid) a.vis.range(a.base_pos + qi, vs, ve);
            float m_used = -INFINITY, l = 0.0f;
            for (int j = lo_t; j < hi_t; ++j) {
                const int k = j - lo_t;
                TRACE_MARK();
                if (!(ok = mbar_wait(s_full(t), (cs + k) & 1, abortp))) break;
                TRACE_ADD(ts_wait);
                if ((warp & 3) == 0) TRACE_EVT(j - lo, 8 + t * 8);
                fence_after_sync();
                uint32_t sr[4][32];
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx) tmem_ld32(tS + cidx * 32, sr[cidx]);
                tmem_wait_ld();
                TRACE_ADD(ts_ld);
                if ((warp & 3) == 0) TRACE_EVT(j - lo, 9 + t * 8);
                const int key0 = j * kTcBN;
                if (key0 < vs || key0 + kTcBN > ve) {
#pragma unroll
                    for (int cidx = 0; cidx < 4; ++cidx)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int key = key0 + cidx * 32 + i;
                            if (key < vs || key >= ve) sr[cidx][i] = 0xff800000u;  // -inf
                        }
                }
                float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx)
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        mxa = max3(mxa, __uint_as_float(sr[cidx][i]), __uint_as_float(sr[cidx][i + 1]));
                        mxb = max3(mxb, __uint_as_float(sr[cidx][i + 2]), __uint_as_float(sr[cidx][i + 3]));
                        mxc = max3(mxc, __uint_as_float(sr[cidx][i + 4]), __uint_as_float(sr[cidx][i + 5]));
                        mxd = max3(mxd, __uint_as_float(sr[cidx][i + 6]), __uint_as_float(sr[cidx][i + 7]));
                    }
                const float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
                TRACE_ADD(ts_max);
                if ((warp & 3) == 0) TRACE_EVT(j - lo, 10 + t * 8);
                // lazy rescale of the running output
                const bool need = mx > m_used + thr;
                float alpha = 1.0f;
                if (need) {
                    alpha = ex2((m_used - mx) * c);  // 0 when nothing was accumulated yet
                    m_used = mx;
                }
                if (k > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                    for (int cidx = 0; cidx < D / 32; ++cidx) {  // rare path, kept small
                        uint32_t orow[32];
                        tmem_ld32(tO + cidx * 32, orow);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                        tmem_st32(tO + cidx * 32, orow);
                    }
                }
                l *= alpha;
                TRACE_ADD(ts_resc);
                if ((warp & 3) == 0) TRACE_EVT(j - lo, 11 + t * 8);
                const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
                const float neg = -mref * c;
                // p = 2^(s * c - m * c): one packed FMA per two scores, sums kept as packed pairs. Two variants were
                // measured and dropped: ex2.approx.f16x2 (half-precision pairs) made this phase slower, and writing
                // P as f16 against a bf16 V is an illegal instruction (A and B of one MMA share the 16-bit type).
                const uint64_t c2 = pack_f32x2(c, c), neg2 = pack_f32x2(neg, neg);
                uint64_t sum_a = 0ull, sum_b = 0ull;  // bit pattern of (0.0f, 0.0f)
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const uint64_t ta = fma_f32x2(pack_f32x2(__uint_as_float(sr[cidx][2 * i]), __uint_as_float(sr[cidx][2 * i + 1])), c2, neg2);
                        const uint64_t tb = fma_f32x2(pack_f32x2(__uint_as_float(sr[cidx][2 * i + 2]), __uint_as_float(sr[cidx][2 * i + 3])), c2, neg2);
                        float x0, x1, p2, p3;
                        unpack_f32x2(ta, x0, x1);
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        if (kExpPolyMask & (1 << ((i >> 1) & 3))) {
                            ex2_poly_x2(tb, p2, p3);
                        } else {
                            float x2, x3;
                            unpack_f32x2(tb, x2, x3);
                            p2 = ex2(x2);
                            p3 = ex2(x3);
                        }
                        sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
                        sum_b = add_f32x2(sum_b, pack_f32x2(p2, p3));
                        __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1);
                        __nv_bfloat162 pb = __floats2bfloat162_rn(p2, p3);
                        pk[i] = *reinterpret_cast<uint32_t*>(&pa);
                        pk[i + 1] = *reinterpret_cast<uint32_t*>(&pb);
                    }
                    tmem_st16(tS + cidx * 16, pk);
                    if (cidx == 1) {
                        // keys 0-63 of P_t are in TMEM: their half of P V starts while the other half is computed
                        tmem_wait_st();
                        fence_before_sync();
                        mbar_arrive(p_half(t, 0));
                    }
                }
                {
                    float s0, s1;
                    unpack_f32x2(add_f32x2(sum_a, sum_b), s0, s1);
                    l += s0 + s1;
                }
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(p_half(t, 1));
                TRACE_ADD(ts_exp);
                if ((warp & 3) == 0) TRACE_EVT(j - lo, 12 + t * 8);
            }
            if (!ok) break;
            cs += n_t;
            // epilogue: O_t leaves TMEM as soon as its last P V has landed, then the next item may overwrite it
            TRACE_MARK();
            if (!(ok = mbar_wait(o_final(t), it & 1, abortp))) break;
            TRACE_ADD(ts_ofin);
            fence_after_sync();
            if (n_t > 0) {
                // The rows leave through a per-warp staging area: a thread (one query row) lays 32 output columns
                // down as 128 bytes, 16-byte pieces XOR-swizzled by the row so that the eight rows of a quarter
                // warp hit different banks; the warp then reads the area back four rows at a time and stores
                // whole 128-byte lines. One thread per row storing 16-byte pieces 16 KB apart cost a cache-line
                // wavefront per lane and instruction, 3-4 us per item during which the tile's pipeline stood still.
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                const void* grow = nullptr;
                if (a.gate && valid)
                    grow = static_cast<const unsigned char*>(a.gate) +
                           ((int64_t)qi * Hq + w.h) * a.gate_head_stride * (a.gate_bf16 ? 2 : 4);
                const uint32_t stage = sOut + (uint32_t)warp * 4096u;
                const int row_w = w.q_row0 + t * kTcBM + (warp & 3) * 32;   // first row of this warp
                const int sub_row = lane >> 3, piece = lane & 7;
                // (a rolled loop: this code runs once per item, and unrolled it missed the instruction cache line after
                // line; the next item's first P V into O_t is a whole softmax tile away, so O_t may stay until the end)
#pragma unroll 1
                for (int cidx = 0; cidx < D / 32; ++cidx) {
                    uint32_t orow[32];
                    tmem_ld32(tO + cidx * 32, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o4 = make_float4(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv,
                                                __uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
                        if (grow) o4 = prefill_gate4(o4, grow, a.gate_bf16, cidx * 32 + i);
                        const uint32_t dst = stage + lane * 128u + (uint32_t)(((i >> 2) ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(o4.x), "f"(o4.y), "f"(o4.z), "f"(o4.w) : "memory");
                    }
                    __syncwarp();
#pragma unroll
                    for (int k4 = 0; k4 < 8; ++k4) {
                        const int rr = k4 * 4 + sub_row;
                        float4 o4;
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(o4.x), "=f"(o4.y), "=f"(o4.z), "=f"(o4.w)
                                     : "r"(stage + rr * 128u + (uint32_t)((piece ^ (rr & 7)) << 4)));
                        if (row_w + rr < a.m)
                            *reinterpret_cast<float4*>(a.out + ((int64_t)(row_w + rr) * Hq + w.h) * D + cidx * 32 + piece * 4) = o4;
                    }
                    __syncwarp();
                }
                fence_before_sync();
                mbar_arrive(o_free(t));
            } else {
                mbar_arrive(o_free(t));
            }
            TRACE_ADD(ts_epi);
#ifdef GGR_TC_TRACE
            ++ts_items;
#endif
        }
#ifdef GGR_TC_TRACE
        if (blockIdx.x == 0 && a.trace && (tid & 127) == 0) {
            long long* o = a.trace + 8 + t * 8;
            o[0] = clock64() - ts_t0; o[1] = ts_wait; o[2] = ts_ld; o[3] = ts_max; o[4] = ts_resc; o[5] = ts_exp; o[6] = cs;
            long long* o2 = a.trace + 128 + t * 4;
            o2[0] = ts_item; o2[1] = ts_ofin; o2[2] = ts_epi; o2[3] = ts_items;
        }
#endif
    }

    // ---------------- common tail ----------------
    if (s_abort) {
        // let copies that are still in flight land before shared memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 9) tmem_dealloc(tmem, 512);
    if (tid == 0) {
        if (s_abort && a.err) atomicExch(a.err, 1);
        // the last CTA to leave rewinds the work counter for the next launch on this stream
        __threadfence();
        if (atomicAdd(a.sched + 1, 1) == (int)gridDim.x - 1) {
            a.sched[0] = 0;
            a.sched[1] = 0;
            __threadfence();
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------

inline bool prefill_tc_shape_ok(int fmt, int D) { return fmt == KV_BF16 && (D == 64 || D == 128); }

inline bool prefill_tc_usable(int impl, int fmt, int D, int /*G*/) {
    if (impl == 1 /* GGR_IMPL_SIMT */) return false;
    return prefill_tc_shape_ok(fmt, D);
}

inline size_t prefill_tc_smem(int D) { return (size_t)6 * (D / 64) * 128 * 128 + 8 * 4096 + 1024; }

template <int D>
inline int launch_prefill_tc_inst(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                  const PrefillTcArgs& a, int device, int sm_count, cudaStream_t stream,
                                  std::string* msg) {
    static KernelSmemSetup setup;
    const size_t smem = prefill_tc_smem(D);
    {
        const cudaError_t e = setup.ensure(prefill_tc_kernel<D>, device, 0, (int)smem);
        if (e != cudaSuccess) {
            *msg = std::string("prefill kernel attribute: ") + cudaGetErrorString(e);
            return 2;
        }
    }
    if (sm_count <= 0 || !a.sched) {
        *msg = "prefill kernel: no SM count or no scheduler counters";
        return 2;
    }
    PrefillTcArgs args = a;
    const int n_pairs = (a.m + 2 * kTcBM - 1) / (2 * kTcBM);
    args.n_items = n_pairs * a.kv.Hq;
    const int grid = args.n_items < sm_count ? args.n_items : sm_count;  // one persistent CTA per SM
    cudaError_t e;
    if (args.dependent) {
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(grid);
        lc.blockDim = dim3(kTcThreads);
        lc.dynamicSmemBytes = smem;
        lc.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        e = cudaLaunchKernelEx(&lc, prefill_tc_kernel<D>, tq, tk, tv, args);
    } else {
        prefill_tc_kernel<D><<<grid, kTcThreads, smem, stream>>>(tq, tk, tv, args);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        *msg = std::string("prefill kernel launch: ") + cudaGetErrorString(e);
        return 2;
    }
    return 0;
}

// tk / tv describe the whole K and V cache arrays as [rows][kv_dim].
inline int launch_prefill_tc(const PrefillTcArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, int device,
                             int sm_count, cudaStream_t stream, std::string* msg) {
    CUtensorMap tq;
    if (!make_tmap_bf16(&tq, a.q, (uint64_t)a.kv.Hq * a.kv.D, (uint64_t)a.m)) {
        *msg = "cuTensorMapEncodeTiled failed for the query tensor";
        return 2;
    }
    switch (a.kv.D) {
        case 64: return launch_prefill_tc_inst<64>(tq, tk, tv, a, device, sm_count, stream, msg);
        case 128: return launch_prefill_tc_inst<128>(tq, tk, tv, a, device, sm_count, stream, msg);
        default: *msg = "no tensor-core prefill kernel for this head_dim"; return 5;
    }
}

}  // namespace ggr
