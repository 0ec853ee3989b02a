// Tensor-core prefill for head_dim 256 (Gemma-3-shaped layers): same algorithm as prefill_tc_kernel,
// different tiling because the output accumulator alone takes 256 TMEM columns.
//
// One CTA owns ONE 128-row query tile of one query head and walks the visible 64-key tiles:
//   warp 4       TMA producer (K and V tiles of 64 keys into 3-stage rings)
//   warp 5       MMA issuer: S[b] = Q K^T (N = 64) into one of two S buffers, O += P V (N = 256)
//   warps 0-3    softmax, one thread per query row; they also place Q in tensor memory at the start and send the
//                output rows out at the end, both as one bulk copy per row through shared memory (a warp that
//                reads or writes one 16-byte piece per row touches 32 cache lines per instruction: that took
//                3.3 us for Q and 8.2 us for the output of a 28 us CTA)
// TMEM columns: S0 0-63, S1 64-127, O 128-383, Q 384-511 (bf16 pairs, the A operand of Q K^T). With Q in
// shared memory an N = 64 instruction fetched 4 KB of Q and 2 KB of K for 32 cycles of arithmetic and
// ran at the shared-memory rate (48 cycles); from tensor memory only the K fetch remains, and the 64 KB
// of shared memory Q occupied hold a third K / V stage. The score tile of step j+1 is computed while the
// softmax of step j runs. Because QK(j+1) is issued before PV(j), O is still being written when the
// softmax of step j+1 starts: a step that has to rescale O waits for PV(j) (pv_done) first, every other
// step only observes that barrier after its exponentials, where the wait is normally over. P is
// published in two 32-key halves so that P V starts under the second half of the softmax.
// Shared memory: 3 stages of (32 KB K, 32 KB V) = 192 KB; the third stage first holds the staged Q rows, and the
// whole ring holds the output rows once the last MMA has completed. Every wait is bounded.
#pragma once

#include <string>

#include "common.cuh"
#include "prefill_tc.cuh"
#include "sm100_utils.cuh"

namespace ggr {

constexpr int kTwBN = 64;        // keys per tile
constexpr int kTwThreads = 256;  // softmax warpgroup + control warpgroup
constexpr int kTwStages = 3;     // K / V ring depth
constexpr uint32_t kTwTailBytes = 2048;  // room past the last stage for the row pitch of the staged Q tile

template <int D>
__global__ void __launch_bounds__(kTwThreads, 1)
prefill_tc_wide_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, PrefillTcArgs a) {
    using namespace tc;
    constexpr int NBLK = D / 64;
    constexpr uint32_t KBLK = kTwBN * 128;       // [64 rows][128 bytes]
    constexpr uint32_t KV_BYTES = NBLK * KBLK;
    constexpr uint32_t O_COL0 = 128;
    constexpr uint32_t Q_COL0 = O_COL0 + D;      // D / 2 columns of bf16 pairs
    constexpr int NST = kTwStages;
    static_assert(Q_COL0 + D / 2 <= 512, "tensor memory columns");

#ifdef GGR_TC_TRACE
    // wall-clock stamps (ns) of the first and the last CTA of diagnostic builds: trace slots 32.. / 40..
#define TW_STAMP(slot) do { if (a.trace && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) { unsigned long long t_; \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); a.trace[(blockIdx.x == 0 ? 32 : 40) + (slot)] = (long long)t_; } } while (0)
    if (threadIdx.x == 0) TW_STAMP(0);
#else
#define TW_STAMP(slot)
#endif
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[24];  // 23 used
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    // the warp index goes through a broadcast so that the compiler knows the role branches are warp-uniform
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES;   // K tile, then V tile
    const uint32_t sK = smem_base;                   // stage s at + s * STAGE_BYTES
    const uint32_t sV = smem_base + KV_BYTES;
    // Rows staged for one-thread-per-row access are pitched 16 bytes past a multiple of 128, which spreads the
    // eight rows of a quarter warp over all banks.
    constexpr uint32_t Q_PITCH = D * 2 + 16, O_PITCH = D * 4 + 16;
    const uint32_t sQst = smem_base + (NST - 1) * STAGE_BYTES;   // last stage (+ the tail of the buffer)
    static_assert(kTcBM * Q_PITCH <= STAGE_BYTES + kTwTailBytes, "staged Q rows");
    static_assert(kTcBM * O_PITCH <= NST * STAGE_BYTES, "staged output rows");

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0;
    auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (4 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (7 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (10 + s); };
    auto s_full = [&](int b) { return bar0 + 8u * (13 + b); };
    // P and "P V landed" barriers exist once per score buffer. Q K^T of step n + 1 is issued before P V of step n,
    // so the softmax warps can be a whole step ahead of the MMA warp: with one barrier for both buffers they could
    // complete its phase n + 1 before the MMA warp had looked at phase n, and a parity wait cannot tell phase n
    // from phase n + 2 (the kernel then sat in a wait until its bound ran out). A buffer's own barrier cannot run
    // ahead: its next phase needs the next-but-one score tile, which the MMA warp issues after it has seen this one.
    auto p_half = [&](int buf, int half) { return bar0 + 8u * (15 + 2 * buf + half); };  // P keys 0-31 / 32-63 stored
    auto pv_done = [&](int buf) { return bar0 + 8u * (19 + buf); };
    const uint32_t o_final = bar0 + 8u * 21;
    const uint32_t q_staged = bar0 + 8u * 22;   // the bulk copies of the Q rows have landed

    const int Hq = a.kv.Hq, G = a.kv.G;
    const int n_tiles = (a.m + kTcBM - 1) / kTcBM;
    const int qt = n_tiles - 1 - (int)(blockIdx.x / Hq);  // long (late) tiles first
    const int h = blockIdx.x % Hq;
    const int kvh = h / G;
    const int q_row0 = qt * kTcBM;

    int lo, hi;
    {
        const int r1 = min(a.m, q_row0 + kTcBM) - 1;
        int vs0, ve0, vs1, ve1;
        a.vis.range(a.base_pos + q_row0, vs0, ve0);
        a.vis.range(a.base_pos + r1, vs1, ve1);
        lo = min(vs0, vs1) / kTwBN;
        hi = (max(ve0, ve1) + kTwBN - 1) / kTwBN;
    }

    if (tid == 0) {
        s_abort = 0;
        mbar_init(q_full, kTcBM);
        for (int s = 0; s < NST; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full(s), 1);
            mbar_init(p_half(s, 0), kTcBM);
            mbar_init(p_half(s, 1), kTcBM);
            mbar_init(pv_done(s), 1);
        }
        mbar_init(o_final, 1);
        mbar_init(q_staged, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&s_tmem_base), 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = s_tmem_base;
    volatile int* abortp = &s_abort;
    const int64_t row_base = a.kv.row(a.seq, a.layer, 0);
    if (threadIdx.x == 0) TW_STAMP(1);
    if (a.dependent) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) TW_STAMP(2);

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 1;  // stage and phase of the ring position: the first pass finds every stage free
            for (int j = lo; j < hi; ++j) {
                const int y = (int)(row_base + (int64_t)j * kTwBN);
                // the last stage holds the staged Q rows until they are in tensor memory
                if (j - lo == NST - 1 && !mbar_wait(q_full, 0, abortp)) break;
                if (!mbar_wait(k_empty(s), ph, abortp)) break;
                mbar_expect_tx(k_full(s), KV_BYTES);
                for (int b = 0; b < NBLK; ++b)
                    tma_load_2d(sK + s * STAGE_BYTES + b * KBLK, &tmK, kvh * D + b * 64, y, k_full(s));
                if (!mbar_wait(v_empty(s), ph, abortp)) break;
                mbar_expect_tx(v_full(s), KV_BYTES);
                for (int b = 0; b < NBLK; ++b)
                    tma_load_2d(sV + s * STAGE_BYTES + b * KBLK, &tmV, kvh * D + b * 64, y, v_full(s));
                if (++s == NST) s = 0, ph ^= 1u;
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (hi > lo) {  // the whole warp runs the loop, one elected lane issues
            constexpr uint32_t IDESC_QK = idesc_bf16(kTwBN, 0);
            constexpr uint32_t IDESC_PV = idesc_bf16(D, 1);
            const uint64_t dK = smem_desc(sK, 16, 1024), dV = smem_desc(sV, KBLK, 1024);
            const uint32_t tmem = __shfl_sync(0xffffffffu, s_tmem_base, 0);  // shadows the CTA-wide copy: provably uniform
            auto issue_qk = [&](int buf, int s) {
                const uint64_t b0 = dK + (uint64_t)((s * STAGE_BYTES) >> 4);
                const uint32_t d = tmem + buf * kTwBN;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    mma_ts_e(d, tmem + Q_COL0 + ks * 8, b0 + (uint64_t)(((ks >> 2) * KBLK + (ks & 3) * 32) >> 4), IDESC_QK,
                             ks > 0 ? 1u : 0u);
                }
            };
            auto issue_pv_half = [&](int buf, int s, int half, bool accumulate) {
                const uint64_t b0 = dV + (uint64_t)((s * STAGE_BYTES) >> 4);
                const uint32_t p0 = tmem + buf * kTwBN;
#pragma unroll
                for (int kk = 0; kk < kTwBN / 32; ++kk) {
                    const int ks = half * (kTwBN / 32) + kk;
                    mma_ts_e(tmem + O_COL0, p0 + ks * 8, b0 + (uint64_t)((ks * 16 * 128) >> 4), IDESC_PV, (accumulate || ks > 0) ? 1u : 0u);
                }
            };
#ifdef GGR_TC_TRACE
            long long tr_v = 0, tr_p0 = 0, tr_k = 0, tr_issue = 0, tr_issue_qk = 0, tr_t0 = clock64(), tr_x;
#endif
            bool ok = mbar_wait_warp(q_full, 0, abortp);
            if (ok) ok = mbar_wait_warp(k_full(0), 0, abortp);
            if (ok) {
                fence_after_sync();
                issue_qk(0, 0);
                mma_commit_e(s_full(0));
                mma_commit_e(k_empty(0));
            }
            int s = 0;
            uint32_t ring_ph = 0;  // ring stage of step n and the phase its "full" barriers complete in this pass
            for (int j = lo; ok && j < hi; ++j) {
                const int n = j - lo;
                const int s1 = s + 1 == NST ? 0 : s + 1;
                const uint32_t ring_ph1 = s + 1 == NST ? ring_ph ^ 1u : ring_ph;
                TRACE_MARK();
                if (j + 1 < hi) {
                    if (!(ok = mbar_wait_warp(k_full(s1), ring_ph1, abortp))) break;
                    TRACE_ADD(tr_k);
                    fence_after_sync();
                    issue_qk((n + 1) & 1, s1);
                    mma_commit_e(s_full((n + 1) & 1));
                    mma_commit_e(k_empty(s1));
                    TRACE_ADD(tr_issue_qk);
                }
                if (!(ok = mbar_wait_warp(v_full(s), ring_ph, abortp))) break;
                TRACE_ADD(tr_v);
                if (!(ok = mbar_wait_warp(p_half(n & 1, 0), (n >> 1) & 1, abortp))) break;
                TRACE_ADD(tr_p0);
                fence_after_sync();
                issue_pv_half(n & 1, s, 0, n > 0);
                if (!(ok = mbar_wait_warp(p_half(n & 1, 1), (n >> 1) & 1, abortp))) break;
                fence_after_sync();
                issue_pv_half(n & 1, s, 1, true);
                mma_commit_e(pv_done(n & 1));
                mma_commit_e(v_empty(s));
                if (j == hi - 1) mma_commit_e(o_final);
                TRACE_ADD(tr_issue);
                s = s1;
                ring_ph = ring_ph1;
            }
#ifdef GGR_TC_TRACE
            if (blockIdx.x == 0 && a.trace) {
                a.trace[0] = clock64() - tr_t0; a.trace[1] = tr_v; a.trace[2] = tr_p0; a.trace[3] = 0;
                a.trace[4] = tr_k; a.trace[5] = tr_issue; a.trace[6] = hi - lo; a.trace[7] = tr_issue_qk;
            }
#endif
        }
    } else if (warp < 4) {
        // ---------------- softmax: one thread per query row ----------------
        const int row = warp * 32 + lane;
        const int qi = q_row0 + row;
        const bool valid = qi < a.m;
        int vs = 0, ve = 0;
        if (valid) a.vis.range(a.base_pos + qi, vs, ve);
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const uint32_t tO = tmem + lane_addr + O_COL0;
        const float c = a.score_scale;
        const float thr = 8.0f / c;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
#ifdef GGR_TC_TRACE
        long long ts_wait = 0, ts_ld = 0, ts_max = 0, ts_resc = 0, ts_exp = 0, ts_t0 = clock64(), tr_x;
#endif
        if (hi > lo) {
            // this thread's query row goes to tensor memory as the A operand of Q K^T: lane = row, one column per
            // two consecutive head elements; rows past the end of the chunk are zero
            // (the row comes in as one bulk copy; the thread then reads it back 16 bytes at a time)
            const int n_valid = min(kTcBM, a.m - q_row0);
            if (tid == 0) mbar_expect_tx(q_staged, (uint32_t)n_valid * (uint32_t)(D * 2));
            if (valid) bulk_load(sQst + row * Q_PITCH, a.q + ((int64_t)qi * Hq + h) * D, D * 2, q_staged);
            ok = mbar_wait(q_staged, 0, abortp);
            // (rolled loops here and in the epilogue: unrolled, this once-per-CTA code missed the instruction cache
            // line after line, and the epilogue took 12 us instead of 5)
#pragma unroll 1
            for (int cidx = 0; ok && cidx < D / 64; ++cidx) {
                uint32_t qr[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint4 v4 = make_uint4(0u, 0u, 0u, 0u);
                    if (valid)
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(v4.x), "=r"(v4.y), "=r"(v4.z), "=r"(v4.w)
                                     : "r"(sQst + row * Q_PITCH + (uint32_t)(cidx * 8 + i) * 16u));
                    qr[4 * i] = v4.x, qr[4 * i + 1] = v4.y, qr[4 * i + 2] = v4.z, qr[4 * i + 3] = v4.w;
                }
                tmem_st32(tmem + lane_addr + Q_COL0 + cidx * 32, qr);
            }
            tmem_wait_st();
            fence_before_sync();
            if (ok) mbar_arrive(q_full);
            if (threadIdx.x == 0) TW_STAMP(3);
        }
        for (int j = lo; ok && j < hi; ++j) {
            const int n = j - lo, buf = n & 1;
            const uint32_t tS = tmem + lane_addr + buf * kTwBN;
            TRACE_MARK();
            if (!(ok = mbar_wait(s_full(buf), (n >> 1) & 1, abortp))) break;
            TRACE_ADD(ts_wait);
            fence_after_sync();
            uint32_t sr[2][32];
            tmem_ld32(tS, sr[0]);
            tmem_ld32(tS + 32, sr[1]);
            tmem_wait_ld();
            TRACE_ADD(ts_ld);
            const int key0 = j * kTwBN;
            if (key0 < vs || key0 + kTwBN > ve) {
#pragma unroll
                for (int cidx = 0; cidx < 2; ++cidx)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + cidx * 32 + i;
                        if (key < vs || key >= ve) sr[cidx][i] = 0xff800000u;  // -inf
                    }
            }
            float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
            for (int cidx = 0; cidx < 2; ++cidx)
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    mxa = max3(mxa, __uint_as_float(sr[cidx][i]), __uint_as_float(sr[cidx][i + 1]));
                    mxb = max3(mxb, __uint_as_float(sr[cidx][i + 2]), __uint_as_float(sr[cidx][i + 3]));
                    mxc = max3(mxc, __uint_as_float(sr[cidx][i + 4]), __uint_as_float(sr[cidx][i + 5]));
                    mxd = max3(mxd, __uint_as_float(sr[cidx][i + 6]), __uint_as_float(sr[cidx][i + 7]));
                }
            const float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
            TRACE_ADD(ts_max);
            const bool need = mx > m_used + thr;
            float alpha = 1.0f;
            if (need) {
                alpha = ex2((m_used - mx) * c);
                m_used = mx;
            }
            // O must be quiet before it is rescaled: PV(j-1) was issued after QK(j). A step that rescales waits
            // for it here; the others only keep track of the barrier's phase, after their exponentials, where
            // the wait is normally over already.
            const bool rescale_now = n > 0 && __any_sync(0xffffffffu, need);
            if (rescale_now) {
                if (!(ok = mbar_wait(pv_done((n - 1) & 1), ((n - 1) >> 1) & 1, abortp))) break;
                fence_after_sync();
// (a rolled loop: the path is rare, and straight-line code that runs once costs an instruction-cache miss per line)
#pragma unroll 1
                for (int cidx = 0; cidx < D / 32; ++cidx) {
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
            const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
            const float neg = -mref * c;
            // p = 2^(s * c - m * c): one packed FMA per two scores, sums kept as packed pairs
            const uint64_t c2 = pack_f32x2(c, c), neg2 = pack_f32x2(neg, neg);
            uint64_t sum_a = 0ull, sum_b = 0ull;  // bit pattern of (0.0f, 0.0f)
#pragma unroll
            for (int cidx = 0; cidx < 2; ++cidx) {
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
                if (cidx == 0) {
                    // keys 0-31 of P are in TMEM: their half of P V starts while the other half is computed
                    tmem_wait_st();
                    fence_before_sync();
                    mbar_arrive(p_half(buf, 0));
                }
            }
            {
                float s0, s1;
                unpack_f32x2(add_f32x2(sum_a, sum_b), s0, s1);
                l += s0 + s1;
            }
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(p_half(buf, 1));
            if (n > 0 && !rescale_now && !(ok = mbar_wait(pv_done((n - 1) & 1), ((n - 1) >> 1) & 1, abortp))) break;
            TRACE_ADD(ts_exp);
        }
#ifdef GGR_TC_TRACE
        if (blockIdx.x == 0 && a.trace && tid == 0) {
            long long* o = a.trace + 8;
            o[0] = clock64() - ts_t0; o[1] = ts_wait; o[2] = ts_ld; o[3] = ts_max; o[4] = ts_resc; o[5] = ts_exp; o[6] = hi - lo;
        }
#endif
        if (threadIdx.x == 0) TW_STAMP(4);
        if (ok && hi > lo) ok = mbar_wait(o_final, 0, abortp);
        if (threadIdx.x == 0) TW_STAMP(5);
        if (ok && hi > lo) {
            fence_after_sync();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float* orow_g = a.out + ((int64_t)qi * Hq + h) * D;
            const void* grow = nullptr;
            if (a.gate && valid)
                grow = static_cast<const unsigned char*>(a.gate) +
                       ((int64_t)qi * Hq + h) * a.gate_head_stride * (a.gate_bf16 ? 2 : 4);
            // Every load into the K / V stages has landed and every MMA that read them has completed (o_final): the
            // thread lays its output row down there and sends it out as one bulk copy. A row base that is not
            // 16-byte aligned takes plain stores.
            const bool bulk_out = ((reinterpret_cast<uintptr_t>(orow_g) & 15u) == 0);
            const uint32_t sOrow = smem_base + row * O_PITCH;
#pragma unroll 1
            for (int cidx = 0; cidx < D / 32; ++cidx) {
                uint32_t orow[32];
                tmem_ld32(tO + cidx * 32, orow);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o4 = make_float4(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv,
                                                __uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
                        if (grow) o4 = prefill_gate4(o4, grow, a.gate_bf16, cidx * 32 + i);
                        if (bulk_out)
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(sOrow + (uint32_t)(cidx * 32 + i) * 4u), "f"(o4.x), "f"(o4.y), "f"(o4.z), "f"(o4.w)
                                         : "memory");
                        else
                            *reinterpret_cast<float4*>(orow_g + cidx * 32 + i) = o4;
                    }
                }
            }
            if (valid && bulk_out) {
                fence_smem_to_async_proxy();
                bulk_store(orow_g, sOrow, D * 4);
                bulk_store_commit_and_wait();
            }
        }
    }

    if (threadIdx.x == 0) TW_STAMP(6);
    if (s_abort) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 5) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0) TW_STAMP(7);
    if (tid == 0 && s_abort && a.err) atomicExch(a.err, 1);
}

inline size_t prefill_tc_wide_smem(int D) { return (size_t)(D / 64) * (2 * kTwStages * kTwBN * 128) + kTwTailBytes + 1024; }

// tk / tv: whole cache arrays with a 64 x 64 box; the queries are read with plain loads
inline int launch_prefill_tc_wide(const PrefillTcArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, int device,
                                  cudaStream_t stream, std::string* msg) {
    if (a.kv.D != 256) {
        *msg = "the wide tensor-core prefill kernel is built for head_dim 256";
        return 5;
    }
    static KernelSmemSetup setup;
    const size_t smem = prefill_tc_wide_smem(256);
    {
        const cudaError_t e = setup.ensure(prefill_tc_wide_kernel<256>, device, 0, (int)smem);
        if (e != cudaSuccess) {
            *msg = std::string("prefill kernel attribute: ") + cudaGetErrorString(e);
            return 2;
        }
    }
    const int n_tiles = (a.m + kTcBM - 1) / kTcBM;
    cudaError_t e;
    if (a.dependent) {
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(n_tiles * a.kv.Hq);
        lc.blockDim = dim3(kTwThreads);
        lc.dynamicSmemBytes = smem;
        lc.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        e = cudaLaunchKernelEx(&lc, prefill_tc_wide_kernel<256>, tk, tv, a);
    } else {
        prefill_tc_wide_kernel<256><<<n_tiles * a.kv.Hq, kTwThreads, smem, stream>>>(tk, tv, a);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        *msg = std::string("prefill kernel launch: ") + cudaGetErrorString(e);
        return 2;
    }
    return 0;
}

}  // namespace ggr
