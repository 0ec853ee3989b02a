// Split-KV attention over the cache on CUDA cores (f32 accumulation).
//
// Device counterpart of attention_token (src/engine/runtime/inference.rs:1970-2530):
// one launched item is one query token; a CTA owns (split, kv_head, item) and
// serves all G = n_heads / n_kv_heads query heads of that KV head, so each
// cache byte is read once (the reference re-reads it per query head).
//
// Data movement: every warp runs its own cp.async ring (NST stages of TK keys,
// 16-byte copies straight from the cache rows into shared memory), so loads
// stay in flight while the previous tile is reduced. Scores are reduced across
// the lanes of a key with shuffles; softmax is the online form with base-2
// exponentials; the per-warp states are merged in shared memory, the per-split
// states through a scratch buffer by the last CTA to finish (atomic ticket).
#pragma once

#include "common.cuh"
#include "rope_append.cuh"

namespace ggr {

constexpr int kSimtTK = 16;      // keys per pipeline stage of one warp
constexpr int kSimtWarps = 4;

// Decode fusion: the attention kernel itself rotates q (every CTA, for its own query heads) and the
// CTA whose key range holds the new position rotates k and appends the k / v row slice of its KV head
// before it starts streaming, so a decode step is one launch per layer instead of two.
struct FusedRope {
    int enabled;
    RopeParams rope;
    const float* q_in;  // [items][q_dim] f32, before RoPE
    const float* k_in;  // [items][kv_dim]
    const float* v_in;  // [items][kv_dim]
    int smem_off;       // byte offset of the fusion scratch inside dynamic shared memory
};

// Fused exchange of KV-sequence shards: instead of handing its partial states to a collective, the
// decode kernel stores them straight into the receive slot every rank keeps for this rank (peer memory
// over NVLink, plain stores), and the last (token, kv head) group to finish raises this rank's flag on
// every peer with plain stores; waits on the flags are bounded.
constexpr int kMaxPeers = 8;
struct PeerExchange {
    int enabled;
    int n_ranks, rank;
    float* slot[kMaxPeers];    // rank r's receive slot for this rank's states: [B][Hq][D + 2]
    int* flag[kMaxPeers];      // rank r's flag word for this rank
    int epoch;                 // value the flags take when this step's states are complete
    unsigned* done_counter;    // local count of finished (token, kv head) groups, zero between launches
    int groups_total;
};

struct AttnArgs {
    KvView kv;
    Items items;
    Visibility vis;
    int layer;
    const float* q;       // [items][q_dim], rotated (and pre-scaled where the mode says so)
    float score_scale;    // (1/sqrt(D) or 1) * log2(e), folded into q
    int n_split;
    float* part;          // scratch [items][Hq][n_split][D + 2]: o (un-normalised), m, l
    unsigned* counters;   // scratch [items][Hkv] tickets, zero between launches
    float* out;           // [items][q_dim] final output, or null
    float* partial_out;   // [items][Hq][D + 2] (o / l, m, l) for cross-rank merging, or null
    int shard_count;      // positions held locally
    int stage_bytes;      // bytes of one ring stage of one warp
    int tile_stages;      // ring stages of the CTA-tile kernel (1 or 2)
    int* err;             // raised when a bounded wait runs out (kernels that wait on mbarriers)
    FusedRope fused;
    PeerExchange px;
    // optional output gate (src/engine/runtime/inference.rs:3509-3519): head h of item i at
    // gate + (i * Hq + h) * gate_head_stride; final outputs become finite_or_zero(o * sigmoid(gate))
    const float* gate;
    int gate_head_stride;
#ifdef GGR_TC_TRACE
    long long* trace;     // per-CTA phase time stamps (diagnostic builds only)
#endif
};

// phase time stamps of diagnostic builds: slot k of this CTA's row in a.trace
#ifdef GGR_TC_TRACE
#define DECODE_STAMP(k)                                                                                      \
    do {                                                                                                     \
        if (threadIdx.x == 0 && a.trace) {                                                                   \
            long long t_;                                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                           \
            a.trace[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (k)] = t_;        \
        }                                                                                                    \
    } while (0)
#else
#define DECODE_STAMP(k)
#endif

inline size_t fused_rope_smem_bytes(const KvView& kv, int rope_half) {
    return (size_t)(2 * rope_half + kv.G * kv.D + 2 * kv.kv_dim + 32) * sizeof(float);
}

// Returns the rotated (and pre-scaled) query heads of this CTA's KV head in shared memory.
// `owner` is CTA-uniform: this CTA's key range holds `pos`, so it appends the row first.
__device__ __forceinline__ const float* fused_rope_prologue(const AttnArgs& a, int item, int kvh, int seq, int pos,
                                                            bool owner, unsigned char* smem_base) {
    const RopeParams& rp = a.fused.rope;
    const int D = a.kv.D, G = a.kv.G, Hq = a.kv.Hq, kv_dim = a.kv.kv_dim, half = rp.rope_half;
    const int tid = threadIdx.x, nt = blockDim.x;
    float* cs = reinterpret_cast<float*>(smem_base + a.fused.smem_off);
    float* sn = cs + half;
    float* qs = sn + half;
    float* krow = qs + G * D;
    float* vrow = krow + kv_dim;
    float* red = vrow + kv_dim;
    // The raw q (and, in the owner CTA, k / v) values travel to shared memory with cp.async while the angles
    // are computed, so the prologue costs one round trip to memory instead of two; the rotation then works
    // pairwise in place, with the same separately rounded products as rope_elem.
    const int64_t qb = ((int64_t)item * Hq + (int64_t)kvh * G) * D;
    const int64_t kb = (int64_t)item * kv_dim;
    const bool whole = a.kv.fmt == KV_Q8_ROW;  // the row scale spans all KV heads
    const int e0 = whole ? 0 : kvh * D, e1 = whole ? kv_dim : (kvh + 1) * D;
    {
        const bool al16 = ((reinterpret_cast<uintptr_t>(a.fused.q_in) | reinterpret_cast<uintptr_t>(a.fused.k_in) |
                            reinterpret_cast<uintptr_t>(a.fused.v_in)) & 15) == 0 && (half & 3) == 0;
        auto stage = [&](float* dst, const float* src, int n) {
            if (al16) {
                for (int i = tid * 4; i < n; i += nt * 4) cp_async_16(smem_u32(dst + i), src + i, 16);
            } else {
                for (int i = tid; i < n; i += nt) cp_async_4(smem_u32(dst + i), src + i, 4);
            }
        };
        stage(qs, a.fused.q_in + qb, G * D);
        if (owner) {
            stage(krow + e0, a.fused.k_in + kb + e0, e1 - e0);
            stage(vrow + e0, a.fused.v_in + kb + e0, e1 - e0);
        }
        cp_async_commit();
    }
    for (int i = tid; i < half; i += nt) {
        const int axis = rope_axis(rp.layout, i, rp.sections);
        int coord = pos;
        if (rp.has_plan) coord = pos < rp.plan_len ? rp.plan[pos * 3 + axis] : rp.next_text + (pos - rp.plan_len);
        const float val = __fmul_rn(__fmul_rn((float)coord, rp.freqs[i]), rp.fscale);
        float sv, cv;
        sincosf(val, &sv, &cv);
        cs[i] = cv;
        sn[i] = sv;
    }
    cp_async_wait<0>();
    __syncthreads();
    auto rotate_heads = [&](float* x, int n_heads, bool prescale) {
        for (int p = tid; p < n_heads * half; p += nt) {
            const int g = p / half, j = p - g * half;
            const int i0 = rp.style == 0 ? j : 2 * j, i1 = rp.style == 0 ? j + half : 2 * j + 1;
            float* xh = x + g * D;
            const float v0 = xh[i0], v1 = xh[i1];
            float r0 = __fsub_rn(__fmul_rn(v0, cs[j]), __fmul_rn(v1, sn[j]));
            float r1 = __fadd_rn(__fmul_rn(v0, sn[j]), __fmul_rn(v1, cs[j]));
            if (prescale) {
                r0 = __fmul_rn(r0, rp.q_prescale);
                r1 = __fmul_rn(r1, rp.q_prescale);
            }
            xh[i0] = r0;
            xh[i1] = r1;
        }
        if (prescale) {
            const int tail = D - rp.rope_dim;  // elements beyond the rotated span are only scaled
            for (int p = tid; p < n_heads * tail; p += nt) {
                const int g = p / tail, i = rp.rope_dim + (p - g * tail);
                x[g * D + i] = __fmul_rn(x[g * D + i], rp.q_prescale);
            }
        }
    };
    rotate_heads(qs, G, rp.do_prescale != 0);
    if (owner) {
        rotate_heads(krow + e0, (e1 - e0) / D, false);
        __syncthreads();
        const int64_t r = a.kv.row(seq, a.layer, pos);
        const int64_t off = r * kv_dim + (int64_t)kvh * D;
        const float* kh = krow + kvh * D;
        const float* vh = vrow + kvh * D;
        if (a.kv.fmt == KV_F32) {
            float* kc = reinterpret_cast<float*>(a.kv.k) + off;
            float* vc = reinterpret_cast<float*>(a.kv.v) + off;
            for (int i = tid; i < D; i += nt) {
                kc[i] = kh[i];
                vc[i] = vh[i];
            }
        } else if (a.kv.fmt == KV_BF16) {
            __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(a.kv.k) + off;
            __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(a.kv.v) + off;
            for (int i = tid; i < D; i += nt) {
                kc[i] = __float2bfloat16_rn(kh[i]);
                vc[i] = __float2bfloat16_rn(vh[i]);
            }
        } else if (a.kv.fmt == KV_Q8_ROW) {
            float mk = 0.0f, mv = 0.0f;
            for (int idx = tid; idx < kv_dim; idx += nt) {
                mk = fmaxf(mk, fabsf(krow[idx]));
                mv = fmaxf(mv, fabsf(vrow[idx]));
            }
            mk = warp_max(mk);
            mv = warp_max(mv);
            if ((tid & 31) == 0) {
                red[tid >> 5] = mk;
                red[16 + (tid >> 5)] = mv;
            }
            __syncthreads();
            mk = 0.0f;
            mv = 0.0f;
            for (int w = 0; w < (nt >> 5); ++w) {
                mk = fmaxf(mk, red[w]);
                mv = fmaxf(mv, red[16 + w]);
            }
            const float invk = mk == 0.0f ? 0.0f : __fdiv_rn(127.0f, mk);
            const float invv = mv == 0.0f ? 0.0f : __fdiv_rn(127.0f, mv);
            int8_t* kc = reinterpret_cast<int8_t*>(a.kv.k) + off;
            int8_t* vc = reinterpret_cast<int8_t*>(a.kv.v) + off;
            for (int i = tid; i < D; i += nt) {
                kc[i] = mk == 0.0f ? (int8_t)0 : q8_code(kh[i], invk);
                vc[i] = mv == 0.0f ? (int8_t)0 : q8_code(vh[i], invv);
            }
            if (tid == 0) {  // every KV head's owner CTA writes the same two values
                a.kv.ks[r] = mk == 0.0f ? 1.0f : __fdiv_rn(mk, 127.0f);
                a.kv.vs[r] = mv == 0.0f ? 1.0f : __fdiv_rn(mv, 127.0f);
            }
        } else {  // KV_Q8_BLOCK32: the blocks of this head
            const int nb = kv_dim / 32, nbh = D / 32;
            int8_t* kc = reinterpret_cast<int8_t*>(a.kv.k) + off;
            int8_t* vc = reinterpret_cast<int8_t*>(a.kv.v) + off;
            const int lane = tid & 31, warp = tid >> 5, nwp = nt >> 5;
            for (int b = warp; b < nbh; b += nwp) {
                const float xk = kh[b * 32 + lane], xv = vh[b * 32 + lane];
                const float mk = warp_max(fabsf(xk)), mv = warp_max(fabsf(xv));
                const float invk = mk == 0.0f ? 0.0f : __fdiv_rn(127.0f, mk);
                const float invv = mv == 0.0f ? 0.0f : __fdiv_rn(127.0f, mv);
                kc[b * 32 + lane] = mk == 0.0f ? (int8_t)0 : q8_code(xk, invk);
                vc[b * 32 + lane] = mv == 0.0f ? (int8_t)0 : q8_code(xv, invv);
                if (lane == 0) {
                    a.kv.ks[r * nb + kvh * nbh + b] = mk == 0.0f ? 1.0f : __fdiv_rn(mk, 127.0f);
                    a.kv.vs[r * nb + kvh * nbh + b] = mv == 0.0f ? 1.0f : __fdiv_rn(mv, 127.0f);
                }
            }
        }
        __threadfence();
    }
    __syncthreads();
    // the appended row is read back through cp.async / TMA by this CTA
    if (owner) asm volatile("fence.proxy.async;" ::: "memory");
    return qs;
}

// sigmoid_mul_inplace + sanitize_finite_inplace of one element (src/engine/kernels/math.rs:399-402, :458-462)
__device__ __forceinline__ float gated_output(float o, float gate) {
    const float s = 1.0f / (1.0f + expf(-gate));
    const float r = o * s;
    return isfinite(r) ? r : 0.0f;
}

// Writes one head's merged state: the final output row, a (o / l, m, l)
// partial for cross-rank merging, or nothing when a later stage will.
__device__ __forceinline__ void store_final(const AttnArgs& a, int item, int h, int d, float o, float ms, float ls) {
    const int D = a.kv.D, Hq = a.kv.Hq;
    const float inv = ls > 0.0f ? 1.0f / ls : 0.0f;
    if (a.px.enabled) {
        const int64_t o_idx = ((int64_t)item * Hq + h) * (D + 2);
        const float val = o * inv;
        for (int r = 0; r < a.px.n_ranks; ++r) {
            float* po = a.px.slot[r] + o_idx;
            po[d] = val;
            if (d == 0) {
                po[D] = ms;
                po[D + 1] = ls;
            }
        }
    } else if (a.partial_out) {
        float* po = a.partial_out + ((int64_t)item * Hq + h) * (D + 2);
        po[d] = o * inv;
        if (d == 0) {
            po[D] = ms;
            po[D + 1] = ls;
        }
    } else {
        float r = o * inv;
        if (a.gate) r = gated_output(r, a.gate[((int64_t)item * Hq + h) * a.gate_head_stride + d]);
        a.out[((int64_t)item * Hq + h) * D + d] = r;
    }
}

// Merges the per-warp online-softmax states of a CTA (wacc [nw][RS][D] un-normalised,
// wm / wl [nw][RS]) for heads g0 .. g0+gn-1 of this KV head and stores them: final
// when the launch has one split, else into the split scratch.
__device__ __forceinline__ void cta_merge_store(const AttnArgs& a, const float* wacc, float* wm, float* wl, int nw,
                                                int RS, int g0, int gn, int item, int kvh, int split, int ld = 0) {
    if (ld == 0) ld = a.kv.D;  // row stride of wacc (the tensor-core kernels pad it against bank conflicts)
    const int D = a.kv.D, G = a.kv.G, Hq = a.kv.Hq;
    // one thread per head turns the warps' maxima into weights once (wm <- 2^(m_w - max), wl[g] <- merged l,
    // wx[g] <- max), so the per-element loop below is a plain weighted sum
    float* wx = wl + nw * RS;
    for (int g = threadIdx.x; g < gn; g += blockDim.x) {
        float ms = -INFINITY;
        for (int w = 0; w < nw; ++w) ms = fmaxf(ms, wm[w * RS + g]);
        float ls = 0.0f;
        for (int w = 0; w < nw; ++w) {
            const float mw = wm[w * RS + g];
            const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - ms);
            ls += f * wl[w * RS + g];
            wm[w * RS + g] = f;
        }
        wl[g] = ls;
        wx[g] = ms;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gn * D; idx += blockDim.x) {
        const int g = idx / D, d = idx - g * D;
        float o = 0.0f;
        for (int w = 0; w < nw; ++w) o = fmaf(wm[w * RS + g], wacc[(w * RS + g) * ld + d], o);
        const float ms = wx[g], ls = wl[g];
        const int h = kvh * G + g0 + g;
        if (a.n_split == 1) {
            store_final(a, item, h, d, o, ms, ls);
        } else {
            float* pp = a.part + (((int64_t)item * Hq + h) * a.n_split + split) * (D + 2);
            pp[d] = o;
            if (d == 0) {
                pp[D] = ms;
                pp[D + 1] = ls;
            }
        }
    }
}

// Start of a kernel that feeds the fused shard exchange: lets the merge kernel enqueued behind it (launched with
// programmatic stream serialisation) become resident once every CTA of this grid has started, so that its launch
// and its wait for the peers' flags overlap this grid's work. A no-op for every other launch.
__device__ __forceinline__ void peer_allow_dependents(const AttnArgs& a) {
    if (a.px.enabled) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Called by the CTA that stored the final states of a (token, kv head) group. When every group of the
// launch has finished, this rank's flag is raised on all peers (system-scope release after the stores).
__device__ __forceinline__ void peer_group_done(const AttnArgs& a) {
    if (!a.px.enabled) return;
    // One system-scope fence per CTA, issued after the CTA barrier by the thread that takes the ticket: the barrier
    // orders every thread's stores before it and the fence is cumulative. (A fence in each of the 256 threads cost
    // 16 us per launch: system-scope fences are served one after the other.)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(a.px.done_counter, 1u);
        if (prev == (unsigned)a.px.groups_total - 1u) {
            // one fence, then relaxed flag stores: a release store per peer is a system-scope fence each, and eight
            // of them in a row cost 8 us at the end of every launch
            __threadfence_system();
            for (int r = 0; r < a.px.n_ranks; ++r) {
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(a.px.flag[r]), "r"(a.px.epoch) : "memory");
            }
            *a.px.done_counter = 0u;  // ready for the next launch
        }
    }
}

// floats the split merge needs behind its weights for the sub-results of warps that share a head
inline size_t split_merge_sub_floats(int G, int D) { return G <= 4 ? (size_t)G * 4 * (D + 2) : 0; }

// The last CTA of a (token, kv head) to arrive (atomic ticket) merges the
// per-split states from the scratch buffer and resets the ticket. `wsm` is
// shared memory for G * n_split weights (the drained ring is reused).
__device__ __forceinline__ void split_merge_store(const AttnArgs& a, int item, int kvh, int* s_last, float* wsm) {
    if (a.n_split == 1) {
        peer_group_done(a);
        return;
    }
    const int D = a.kv.D, G = a.kv.G, Hq = a.kv.Hq, NS = a.n_split;
    // one fence on each side of the ticket, issued by the thread that takes it: the CTA barrier before it orders
    // every thread's stores of this CTA's state ahead of the fence, the barrier after it orders every thread's
    // loads of the other CTAs' states behind it (fences are cumulative)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned prev = atomicAdd(&a.counters[item * a.kv.Hkv + kvh], 1u);
        *s_last = (prev == (unsigned)NS - 1u);
        if (*s_last) __threadfence();
    }
    __syncthreads();
    if (!*s_last) return;
    DECODE_STAMP(5);
    const float* base = a.part + ((int64_t)item * Hq + (int64_t)kvh * G) * NS * (D + 2);
    // One warp per head; this CTA runs alone at the end of the launch and a round trip to the states that other
    // SMs just wrote costs about 1.4 us, so everything is arranged for few dependent round trips: (m, l) of all
    // splits in one lane-strided batch of 8-byte loads, the split outputs in batches of 16 or 32 independent
    // 8-byte loads per lane (rows of D + 2 floats are 8-byte aligned).
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (D == 128) {
        // head_dim 128 (two 64-float spans per lane). Several warps share a head when there are more warps than
        // heads: warp (g, sub) merges the splits sub, sub + wph, ... with its own maximum, so that up to 16 * wph
        // splits travel in one round trip; the outputs of a warp's first 16 splits are requested before their
        // (m, l) pairs, so both arrive together. The sub-results are then folded in shared memory.
        int wph = 1;
        while (wph < 4 && G * wph * 2 <= nwarp && 16 * wph < NS) wph <<= 1;
        float* sub_o = wsm + (size_t)G * 2 * NS;  // [G][wph][D + 2]
        for (int gw = warp; gw < G * wph; gw += nwarp) {
            const int g = gw / wph, sub = gw - g * wph;
            const float* hb = base + (int64_t)g * NS * (D + 2);
            float* w = wsm + (size_t)g * 2 * NS;  // [NS] weights, [NS] l
            const float* pp = hb + 2 * lane;
            float2 xa[16], xb[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int sidx = sub + i * wph;
                const bool in = sidx < NS;
                xa[i] = in ? __ldcg(reinterpret_cast<const float2*>(pp + (int64_t)sidx * (D + 2))) : make_float2(0.0f, 0.0f);
                xb[i] = in ? __ldcg(reinterpret_cast<const float2*>(pp + (int64_t)sidx * (D + 2) + 64)) : make_float2(0.0f, 0.0f);
            }
            float ms = -INFINITY;
            for (int sidx = sub + lane * wph; sidx < NS; sidx += 32 * wph) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(hb + (int64_t)sidx * (D + 2) + D));
                w[sidx] = ml.x;
                w[NS + sidx] = ml.y;
                ms = fmaxf(ms, ml.x);
            }
            ms = warp_max(ms);
            float ls = 0.0f;
            for (int sidx = sub + lane * wph; sidx < NS; sidx += 32 * wph) {
                const float mw = w[sidx];
                const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - ms);
                w[sidx] = f;
                ls += f * w[NS + sidx];
            }
            ls = warp_sum(ls);
            __syncwarp();
            DECODE_STAMP(6);
            float ax = 0.0f, ay = 0.0f, bx = 0.0f, by = 0.0f;
            for (int i0 = 0; sub + i0 * wph < NS; i0 += 16) {
                if (i0 > 0) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int sidx = sub + (i0 + i) * wph;
                        const bool in = sidx < NS;
                        xa[i] = in ? __ldcg(reinterpret_cast<const float2*>(pp + (int64_t)sidx * (D + 2))) : make_float2(0.0f, 0.0f);
                        xb[i] = in ? __ldcg(reinterpret_cast<const float2*>(pp + (int64_t)sidx * (D + 2) + 64))
                                   : make_float2(0.0f, 0.0f);
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int sidx = sub + (i0 + i) * wph;
                    const float f = sidx < NS ? w[sidx] : 0.0f;
                    ax = fmaf(f, xa[i].x, ax);
                    ay = fmaf(f, xa[i].y, ay);
                    bx = fmaf(f, xb[i].x, bx);
                    by = fmaf(f, xb[i].y, by);
                }
            }
            if (wph == 1) {
                const int h = kvh * G + g;
                store_final(a, item, h, 2 * lane, ax, ms, ls);
                store_final(a, item, h, 2 * lane + 1, ay, ms, ls);
                store_final(a, item, h, 2 * lane + 64, bx, ms, ls);
                store_final(a, item, h, 2 * lane + 65, by, ms, ls);
            } else {
                float* so = sub_o + ((size_t)g * wph + sub) * (D + 2);
                *reinterpret_cast<float2*>(so + 2 * lane) = make_float2(ax, ay);
                *reinterpret_cast<float2*>(so + 2 * lane + 64) = make_float2(bx, by);
                if (lane == 0) {
                    so[D] = ms;
                    so[D + 1] = ls;
                }
            }
        }
        if (wph > 1) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
                const int g = idx / D, d = idx - g * D;
                const float* so = sub_o + (size_t)g * wph * (D + 2);
                float ms = -INFINITY;
                for (int q = 0; q < wph; ++q) ms = fmaxf(ms, so[q * (D + 2) + D]);
                float o = 0.0f, ls = 0.0f;
                for (int q = 0; q < wph; ++q) {
                    const float mq = so[q * (D + 2) + D];
                    const float f = (mq == -INFINITY) ? 0.0f : exp2f(mq - ms);
                    o = fmaf(f, so[q * (D + 2) + d], o);
                    ls = fmaf(f, so[q * (D + 2) + D + 1], ls);
                }
                store_final(a, item, kvh * G + g, d, o, ms, ls);
            }
        }
        if (threadIdx.x == 0) a.counters[item * a.kv.Hkv + kvh] = 0u;  // ready for the next launch
        peer_group_done(a);
        return;
    }
    for (int g = warp; g < G; g += nwarp) {
        const float* hb = base + (int64_t)g * NS * (D + 2);
        float* w = wsm + (size_t)g * 2 * NS;  // [NS] weights, [NS] l
        float2 xa[16];
        float ms = -INFINITY;
        for (int sidx = lane; sidx < NS; sidx += 32) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(hb + (int64_t)sidx * (D + 2) + D));
            w[sidx] = ml.x;
            w[NS + sidx] = ml.y;
            ms = fmaxf(ms, ml.x);
        }
        ms = warp_max(ms);
        float ls = 0.0f;
        for (int sidx = lane; sidx < NS; sidx += 32) {
            const float mw = w[sidx];
            const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - ms);
            w[sidx] = f;
            ls += f * w[NS + sidx];
        }
        ls = warp_sum(ls);
        __syncwarp();
        DECODE_STAMP(6);
        for (int d0 = 2 * lane; d0 < D; d0 += 64) {
            const float* pp = hb + d0;
            float ox = 0.0f, oy = 0.0f;
            for (int s0 = 0; s0 < NS; s0 += 16) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    xa[i] = s0 + i < NS ? __ldcg(reinterpret_cast<const float2*>(pp + (int64_t)(s0 + i) * (D + 2)))
                                        : make_float2(0.0f, 0.0f);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float f = s0 + i < NS ? w[s0 + i] : 0.0f;
                    ox = fmaf(f, xa[i].x, ox);
                    oy = fmaf(f, xa[i].y, oy);
                }
            }
            store_final(a, item, kvh * G + g, d0, ox, ms, ls);
            store_final(a, item, kvh * G + g, d0 + 1, oy, ms, ls);
        }
    }
    if (threadIdx.x == 0) a.counters[item * a.kv.Hkv + kvh] = 0u;  // ready for the next launch
    peer_group_done(a);
}

// f32 view of the 8 elements lane j owns in a cache row slice held in shared
// memory. Element ownership: f32 -> {4j..4j+3} and {D/2+4j..D/2+4j+3};
// bf16 / q8 -> {8j..8j+7}.
template <int FMT>
__device__ __forceinline__ void load8(const unsigned char* row, int j, int D, const float* scales, float out[8]) {
    if (FMT == KV_F32) {
        float4 a = *reinterpret_cast<const float4*>(row + (size_t)(4 * j) * 4);
        float4 b = *reinterpret_cast<const float4*>(row + (size_t)(D / 2 + 4 * j) * 4);
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else if (FMT == KV_BF16) {
        uint4 u = *reinterpret_cast<const uint4*>(row + (size_t)j * 16);
        out[0] = __uint_as_float(u.x << 16); out[1] = __uint_as_float(u.x & 0xffff0000u);
        out[2] = __uint_as_float(u.y << 16); out[3] = __uint_as_float(u.y & 0xffff0000u);
        out[4] = __uint_as_float(u.z << 16); out[5] = __uint_as_float(u.z & 0xffff0000u);
        out[6] = __uint_as_float(u.w << 16); out[7] = __uint_as_float(u.w & 0xffff0000u);
    } else {
        uint2 u = *reinterpret_cast<const uint2*>(row + (size_t)j * 8);
        float sc = FMT == KV_Q8_ROW ? scales[0] : scales[j >> 2];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[i] = (float)(signed char)((u.x >> (8 * i)) & 0xff) * sc;
            out[4 + i] = (float)(signed char)((u.y >> (8 * i)) & 0xff) * sc;
        }
    }
}

template <int FMT>
__device__ __forceinline__ int elem_index(int j, int p, int D) {
    if (FMT == KV_F32) return p < 4 ? 4 * j + p : D / 2 + 4 * j + (p - 4);
    return 8 * j + p;
}

// Issues the cp.async copies of one tile (K rows, V rows, scales) into a stage.
template <int FMT>
__device__ __forceinline__ void issue_tile(const AttnArgs& a, unsigned char* stage, int64_t row0, int key0,
                                           int key_end, int kvh, int lane) {
    const int D = a.kv.D, eb = a.kv.elem_bytes;
    const int rowbytes = D * eb;
    const int gran = (rowbytes % 16 == 0) ? 16 : ((rowbytes % 8 == 0) ? 8 : 4);
    const int gpr = rowbytes / gran;
    const int total = kSimtTK * gpr;
    unsigned char* ks = stage;
    unsigned char* vs = stage + kSimtTK * rowbytes;
    const unsigned char* kg = reinterpret_cast<const unsigned char*>(a.kv.k);
    const unsigned char* vg = reinterpret_cast<const unsigned char*>(a.kv.v);
    for (int g = lane; g < total; g += 32) {
        int key = g / gpr, col = g - key * gpr;
        int t = key0 + key;
        int valid = t < key_end;
        int tc = valid ? t : key_end - 1;
        int64_t src = ((row0 + tc) * a.kv.kv_dim + (int64_t)kvh * D) * eb + (int64_t)col * gran;
        uint32_t dk = smem_u32(ks + key * rowbytes + col * gran);
        uint32_t dv = smem_u32(vs + key * rowbytes + col * gran);
        if (gran == 16) {
            cp_async_16(dk, kg + src, valid ? 16 : 0);
            cp_async_16(dv, vg + src, valid ? 16 : 0);
        } else if (gran == 8) {
            cp_async_8(dk, kg + src, valid ? 8 : 0);
            cp_async_8(dv, vg + src, valid ? 8 : 0);
        } else {
            cp_async_4(dk, kg + src, valid ? 4 : 0);
            cp_async_4(dv, vg + src, valid ? 4 : 0);
        }
    }
    if (FMT == KV_Q8_ROW || FMT == KV_Q8_BLOCK32) {
        const int nsh = FMT == KV_Q8_ROW ? 1 : D / 32;     // scales of this head per key
        const int nsr = a.kv.n_scales;                      // scales per cache row
        float* ksc = reinterpret_cast<float*>(stage + 2 * kSimtTK * rowbytes);
        float* vsc = ksc + kSimtTK * nsh;
        for (int g = lane; g < kSimtTK * nsh; g += 32) {
            int key = g / nsh, b = g - key * nsh;
            int t = key0 + key;
            int valid = t < key_end;
            int tc = valid ? t : key_end - 1;
            int64_t si = (row0 + tc) * nsr + (FMT == KV_Q8_ROW ? 0 : (int64_t)kvh * nsh + b);
            cp_async_4(smem_u32(ksc + g), a.kv.ks + si, valid ? 4 : 0);
            cp_async_4(smem_u32(vsc + g), a.kv.vs + si, valid ? 4 : 0);
        }
    }
}

template <int FMT, int GH, int NST>
__global__ void __launch_bounds__(kSimtWarps * 32) attn_simt_kernel(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_score[kSimtWarps][GH][kSimtTK];
    __shared__ int s_last;

    const int D = a.kv.D, G = a.kv.G, Hq = a.kv.Hq;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    // the warp index goes through a broadcast so that the compiler knows everything derived from it (key range,
    // ring addresses, TMA coordinates) is warp-uniform
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nw = blockDim.x >> 5;  // 1, 2 or 4 warps, each with its own ring
    const int rowbytes = D * a.kv.elem_bytes;
    DECODE_STAMP(0);
    peer_allow_dependents(a);

    int seq, pos;
    a.items.get(item, seq, pos);
    int vs, ve;
    a.vis.range(pos, vs, ve);
    // keys this rank holds
    vs = max(vs, a.kv.pos_begin);
    ve = min(ve, a.kv.pos_begin + a.shard_count);
    const int T = max(0, ve - vs);
    const int chunk = (T + a.n_split - 1) / a.n_split;
    const int s0 = vs + split * chunk;
    const int s1 = min(ve, s0 + chunk);
    const int64_t row0 = a.kv.row(seq, a.layer, a.kv.pos_begin);  // cache row of local position 0
    // positions are addressed relative to pos_begin below
    const int k0 = s0 - a.kv.pos_begin, k1 = s1 - a.kv.pos_begin;

    // lanes per key and this lane's place
    int chunks = D / 8;
    int LPK = 1;
    while (LPK < chunks) LPK <<= 1;
    const int KPW = 32 / LPK;
    const int grp = lane / LPK, j = lane - grp * LPK;
    const bool active = j < chunks;
    const int nsh = FMT == KV_Q8_ROW ? 1 : (FMT == KV_Q8_BLOCK32 ? D / 32 : 0);

    unsigned char* ring = smem + (size_t)warp * NST * a.stage_bytes;
    const int n_tiles_total = k1 > k0 ? (k1 - k0 + kSimtTK - 1) / kSimtTK : 0;
    // this warp's tiles: warp, warp + W, ...
    const int my_tiles = n_tiles_total > warp ? (n_tiles_total - warp + nw - 1) / nw : 0;

    // The first tiles are requested before the fused prologue (they do not depend on the query), so the
    // rotation of q and the append hide behind their latency. The one exception is the warp of the owner CTA
    // whose first tiles would hold the row that the prologue is about to append.
    const bool owner = a.fused.enabled && pos >= s0 && pos < s1;
    bool prefetched = true;
    if (owner) {
        const int tile_pos = (pos - s0) / kSimtTK;
        if (tile_pos % nw == warp && tile_pos / nw < NST - 1) prefetched = false;
    }
    if (prefetched) {
#pragma unroll
        for (int s = 0; s < NST - 1; ++s) {
            if (s < my_tiles)
                issue_tile<FMT>(a, ring + (size_t)s * a.stage_bytes, row0, k0 + (warp + s * nw) * kSimtTK, k1, kvh, lane);
            cp_async_commit();
        }
    }
    const float* qsrc = a.q + ((int64_t)item * Hq + (int64_t)kvh * G) * D;
    if (a.fused.enabled) qsrc = fused_rope_prologue(a, item, kvh, seq, pos, owner, smem);
    DECODE_STAMP(1);

    for (int g0 = 0; g0 < G; g0 += GH) {
        float qreg[GH][8], acc[GH][8], m[GH], l[GH];
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.0f;
            const bool hv = g0 + g < G;
            const float* qh = qsrc + (int64_t)(g0 + g) * D;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                acc[g][p] = 0.0f;
                qreg[g][p] = (hv && active) ? qh[elem_index<FMT>(j, p, D)] * a.score_scale : 0.0f;
            }
        }

        // prologue: NST - 1 tiles in flight
        if (!(g0 == 0 && prefetched)) {
#pragma unroll
            for (int s = 0; s < NST - 1; ++s) {
                if (s < my_tiles)
                    issue_tile<FMT>(a, ring + (size_t)s * a.stage_bytes, row0, k0 + (warp + s * nw) * kSimtTK, k1,
                                    kvh, lane);
                cp_async_commit();
            }
        }

        for (int it = 0; it < my_tiles; ++it) {
            cp_async_wait<NST - 2>();
            __syncwarp();
            const unsigned char* stage = ring + (size_t)(it % NST) * a.stage_bytes;
            const unsigned char* kt = stage;
            const unsigned char* vt = stage + kSimtTK * rowbytes;
            const float* ksc = reinterpret_cast<const float*>(stage + 2 * kSimtTK * rowbytes);
            const float* vsc = ksc + kSimtTK * nsh;
            const int key0 = k0 + (warp + it * nw) * kSimtTK;

            // scores of the tile
            for (int kk = grp; kk < kSimtTK; kk += KPW) {
                float kf[8];
                if (active) load8<FMT>(kt + (size_t)kk * rowbytes, j, D, ksc + kk * nsh, kf);
                const bool valid = key0 + kk < k1;
#pragma unroll
                for (int g = 0; g < GH; ++g) {
                    float s = 0.0f;
                    if (active) {
#pragma unroll
                        for (int p = 0; p < 8; ++p) s = fmaf(qreg[g][p], kf[p], s);
                    }
                    for (int o = LPK >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (j == 0) s_score[warp][g][kk] = valid ? s : -INFINITY;
                }
            }
            __syncwarp();
            // tile maximum, probabilities, running sum
            float alpha[GH];
            bool any = false;
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float sv = lane < kSimtTK ? s_score[warp][g][lane] : -INFINITY;
                float mx = warp_max(sv);
                float mn = fmaxf(m[g], mx);
                float p = (mn == -INFINITY) ? 0.0f : exp2f(sv - mn);
                float ps = warp_sum(p);
                alpha[g] = (mn == -INFINITY) ? 1.0f : exp2f(m[g] - mn);
                l[g] = l[g] * alpha[g] + ps;
                m[g] = mn;
                if (lane < kSimtTK) s_score[warp][g][lane] = p;
                any |= (mx != -INFINITY);
            }
            __syncwarp();
#pragma unroll
            for (int g = 0; g < GH; ++g) {
#pragma unroll
                for (int p = 0; p < 8; ++p) acc[g][p] *= alpha[g];
            }
            if (any) {
                for (int kk = grp; kk < kSimtTK; kk += KPW) {
                    float vf[8];
                    if (active) {
                        load8<FMT>(vt + (size_t)kk * rowbytes, j, D, vsc + kk * nsh, vf);
#pragma unroll
                        for (int g = 0; g < GH; ++g) {
                            float p = s_score[warp][g][kk];
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
                        }
                    }
                }
            }
            __syncwarp();
            // refill the stage consumed one iteration ago
            const int nt_ = it + NST - 1;
            if (nt_ < my_tiles)
                issue_tile<FMT>(a, ring + (size_t)(nt_ % NST) * a.stage_bytes, row0,
                                k0 + (warp + nt_ * nw) * kSimtTK, k1, kvh, lane);
            cp_async_commit();
        }
        cp_async_wait<0>();

        // fold the key groups of the warp together
#pragma unroll
        for (int g = 0; g < GH; ++g) {
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float v = acc[g][p];
                for (int o = LPK; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[g][p] = v;
            }
        }
        __syncthreads();  // every warp is done with its ring; reuse it as the merge area
        DECODE_STAMP(2);
        float* wacc = reinterpret_cast<float*>(smem);            // [W][GH][D]
        float* wm = wacc + nw * GH * D;                           // [W][GH]
        float* wl = wm + nw * GH;                                 // [W][GH]
        if (grp == 0 && active) {
#pragma unroll
            for (int g = 0; g < GH; ++g) {
#pragma unroll
                for (int p = 0; p < 8; ++p) wacc[(warp * GH + g) * D + elem_index<FMT>(j, p, D)] = acc[g][p];
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                wm[warp * GH + g] = m[g];
                wl[warp * GH + g] = l[g];
            }
        }
        __syncthreads();
        cta_merge_store(a, wacc, wm, wl, nw, GH, g0, min(GH, G - g0), item, kvh, split);
        __syncthreads();  // merge area is free again before the next head group refills the ring
    }

    DECODE_STAMP(3);
    split_merge_store(a, item, kvh, &s_last, reinterpret_cast<float*>(smem));
    DECODE_STAMP(4);
}

// Merges n_parts partial states [n_parts][items][Hq][D + 2] (o / l, m, l) into out.
__global__ void combine_partials_kernel(const float* parts, int n_parts, int items, int Hq, int D, float* out,
                                        const float* gate, int gate_head_stride) {
    const int h = blockIdx.x, item = blockIdx.y;
    const int64_t stride = (int64_t)items * Hq * (D + 2);
    const float* base = parts + ((int64_t)item * Hq + h) * (D + 2);
    float ms = -INFINITY;
    for (int r = 0; r < n_parts; ++r) ms = fmaxf(ms, base[r * stride + D]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.0f, ls = 0.0f;
        for (int r = 0; r < n_parts; ++r) {
            float mw = base[r * stride + D], lw = base[r * stride + D + 1];
            float f = (mw == -INFINITY) ? 0.0f : lw * exp2f(mw - ms);
            o += f * base[r * stride + d];
            ls += f;
        }
        float r = ls > 0.0f ? o / ls : 0.0f;
        if (gate) r = gated_output(r, gate[((int64_t)item * Hq + h) * gate_head_stride + d]);
        out[((int64_t)item * Hq + h) * D + d] = r;
    }
}

// Merge of the states every rank stored into this rank's receive slots. One lane per CTA first waits
// until all flags carry this step's epoch; the states are read around L1, which may still hold the
// lines of an earlier step. The wait is bounded twice, by wall time (wait_ns on %globaltimer) and by an
// iteration count; when it runs out the kernel stores 1 into the error word, writes zeros and returns.
// A peer may legitimately be one step ahead (it has finished this step and sent the next one into the
// other parity); a flag further ahead means the ranks' step counters disagree: error word 2, zeros.
constexpr int kCombineHeads = 8;  // query heads (warps) per CTA of the exchange merge

__global__ void combine_exchange_kernel(const float* parts, const int* flags, int epoch, int n_parts, int64_t part_stride,
                                        int Hq, int D, float* out, int* err, unsigned long long wait_ns,
                                        const float* gate, int gate_head_stride) {
    __shared__ int s_ok;
    const int item = blockIdx.y;
    if (threadIdx.x < 32) {
        // lane r watches rank r's flag with relaxed loads; one system-scope fence after the last flag has arrived
        // makes the peers' states visible (an acquire load per poll is a fence each: eight flags checked one after
        // the other cost 8 us even when all of them were already set). More than 32 ranks: lanes take several.
        int ok = 1;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int r = threadIdx.x; r < n_parts; r += 32) {
            int seen = 0;
            for (uint32_t it = 0; it < (1u << 24); ++it) {
                asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
                if (seen >= epoch) break;
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (now - t0 > wait_ns) break;
                __nanosleep(100);
            }
            if (seen < epoch) ok = min(ok, 0);
            else if (seen > epoch + 1) ok = -1;
        }
        // worst status over the lanes: -1 (a flag ahead of this step) before 0 (a wait ran out) before 1
        const bool any_ahead = __any_sync(0xffffffffu, ok == -1), any_late = __any_sync(0xffffffffu, ok == 0);
        ok = any_ahead ? -1 : (any_late ? 0 : 1);
        if (threadIdx.x == 0) {
            __threadfence_system();
            s_ok = ok;
            if (ok != 1 && err) atomicExch(err, ok == 0 ? 1 : 2);
        }
    }
    __syncthreads();
    const bool ok = s_ok == 1;
    // one warp per query head (kCombineHeads heads per CTA, so that few CTAs pay the wait and the fence); a lane owns
    // pairs of output elements and fetches them from every rank with independent 8-byte loads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x * kCombineHeads + warp;
    if (h >= Hq) return;
    const float* base = parts + ((int64_t)item * Hq + h) * (D + 2);
    // everything a lane needs is requested before anything is used, so the merge costs one round trip: lane r
    // fetches rank r's (m, l) (at most kMaxPeers ranks), every lane its output pairs of all ranks
    float2 ml = make_float2(-INFINITY, 0.0f);
    if (lane < n_parts) ml = __ldcg(reinterpret_cast<const float2*>(base + lane * part_stride + D));
    for (int d0 = 0; d0 < D / 2; d0 += 64) {
        const int da = d0 + lane, db = d0 + 32 + lane;
        float2 oa[kMaxPeers], ob[kMaxPeers];
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            const bool in = r < n_parts;
            oa[r] = (in && da < D / 2) ? __ldcg(reinterpret_cast<const float2*>(base + r * part_stride) + da) : make_float2(0.0f, 0.0f);
            ob[r] = (in && db < D / 2) ? __ldcg(reinterpret_cast<const float2*>(base + r * part_stride) + db) : make_float2(0.0f, 0.0f);
        }
        const float ms = warp_max(ml.x);
        const float fw = (ml.x == -INFINITY) ? 0.0f : ml.y * exp2f(ml.x - ms);  // weight of rank `lane`
        const float ls = warp_sum(fw);
        float ax = 0.0f, ay = 0.0f, bx = 0.0f, by = 0.0f;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            const float f = __shfl_sync(0xffffffffu, fw, r);
            ax += f * oa[r].x;
            ay += f * oa[r].y;
            bx += f * ob[r].x;
            by += f * ob[r].y;
        }
        const float inv = (ok && ls > 0.0f) ? 1.0f / ls : 0.0f;
        const float* gr = (ok && gate) ? gate + ((int64_t)item * Hq + h) * gate_head_stride : nullptr;
        if (da < D / 2) {
            float rx = ax * inv, ry = ay * inv;
            if (gr) rx = gated_output(rx, gr[2 * da]), ry = gated_output(ry, gr[2 * da + 1]);
            *reinterpret_cast<float2*>(out + ((int64_t)item * Hq + h) * D + 2 * da) = make_float2(rx, ry);
        }
        if (db < D / 2) {
            float rx = bx * inv, ry = by * inv;
            if (gr) rx = gated_output(rx, gr[2 * db]), ry = gated_output(ry, gr[2 * db + 1]);
            *reinterpret_cast<float2*>(out + ((int64_t)item * Hq + h) * D + 2 * db) = make_float2(rx, ry);
        }
    }
}

}  // namespace ggr
