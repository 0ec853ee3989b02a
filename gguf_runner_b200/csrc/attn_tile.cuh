// Split-KV decode attention on CUDA cores with CTA-wide key tiles, for the cache formats and head
// groupings the tensor-core decode kernels do not take (f32 and q8 caches, bf16 with fewer than three
// query heads per KV head) at head_dim 64, 128 or 256.
//
// Device counterpart of attention_token (src/engine/runtime/inference.rs:1970-2530) like
// attn_simt_kernel, with the work laid out for short contexts, where a CTA holds one or two tiles and the
// launch is bound by latency rather than by HBM: a CTA of eight warps owns (split, kv head, item) and
// walks its keys in tiles of 64 (32 for 1 KB rows). Per tile
//   load    all 256 threads copy the K and V rows (and q8 scales) with 16-byte cp.async into rows padded
//           by 16 bytes, so that a lane per key reads its row without bank conflicts;
//   scores  thread = (key, slice of the head): one K slice against the slices of all query heads of the KV
//           head (q is read as a broadcast), partial dots to shared memory;
//   softmax warp g = query head g: sums the partial dots, tile maximum and sum with shuffles, online
//           update of (m, l), probabilities and the rescale factor to shared memory;
//   P V     thread = (4 bytes of the head, key group): accumulators for all query heads in registers.
// Three block barriers per tile instead of a shuffle tree per key; with two or three CTAs per SM the
// phases of different CTAs overlap. RoPE of q, the append of the new row and the split merge are the
// shared ones (fused_rope_prologue, split_merge_store).
#pragma once

#include "attn_simt.cuh"
#include "common.cuh"

namespace ggr {

constexpr int kTileThreads = 256;
constexpr int kTileGH = 8;  // query heads per pass over the keys

template <int FMT, int D>
struct TileGeom {
    static constexpr int EB = FMT == KV_F32 ? 4 : (FMT == KV_BF16 ? 2 : 1);
    static constexpr int ROWB = D * EB;                 // bytes of one head's slice of a cache row
    static constexpr int TK = ROWB <= 512 ? 64 : 32;    // keys per tile
    static constexpr int RS = ROWB + 16;                // padded row stride in shared memory
    static constexpr int GPR = ROWB / 16;               // 16-byte pieces per row
    static constexpr int NC = kTileThreads / TK;        // slices of the head in the score phase
    static constexpr int CD = D / NC;                   // elements per slice
    static constexpr int NSH = FMT == KV_Q8_ROW ? 1 : (FMT == KV_Q8_BLOCK32 ? D / 32 : 0);  // scales per key of this head
    static constexpr int EPT = 4 / EB;                  // head elements per thread in P V (4 bytes)
    static constexpr int DT = D / EPT;                  // threads across the head
    static constexpr int KG = kTileThreads / DT;        // key groups
    static constexpr int KPG = TK / KG;                 // keys per group and tile
    static constexpr int MAT = TK * RS;                 // bytes of one K or V tile
    static constexpr int STAGE = (2 * MAT + 2 * TK * NSH * 4 + 15) / 16 * 16;
    static constexpr int PIECE = 16 / EB;               // elements per 16-byte piece
    static_assert(D == 64 || D == 128 || D == 256, "head_dim");
    static_assert(CD * EB % 16 == 0 && KG >= 1 && TK % KG == 0 && KG * KPG == TK, "tile geometry");
};

// bytes of dynamic shared memory before the fusion scratch: per-head scalars (128 bytes), then the ring, the
// partial dots and the probabilities; the same area later holds the key groups' accumulators [KG][8][D]
template <int FMT, int D>
inline size_t tile_smem_bytes(int nst) {
    using Ge = TileGeom<FMT, D>;
    const size_t body = (size_t)nst * Ge::STAGE + (size_t)(Ge::NC + 1) * kTileGH * Ge::TK * 4;
    const size_t fold = (size_t)Ge::KG * kTileGH * D * 4;
    return 128 + (body > fold ? body : fold);
}

template <int FMT, int D>
__global__ void __launch_bounds__(kTileThreads) attn_tile_kernel(AttnArgs a) {
    using Ge = TileGeom<FMT, D>;
    constexpr int TK = Ge::TK, RS = Ge::RS, NC = Ge::NC, CD = Ge::CD, NSH = Ge::NSH, EPT = Ge::EPT, DT = Ge::DT,
                  KG = Ge::KG, KPG = Ge::KPG, EB = Ge::EB, PIECE = Ge::PIECE;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;

    const int G = a.kv.G, Hq = a.kv.Hq;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nst = a.tile_stages;
    DECODE_STAMP(0);
    peer_allow_dependents(a);

    int seq, pos;
    a.items.get(item, seq, pos);
    int vs, ve;
    a.vis.range(pos, vs, ve);
    vs = max(vs, a.kv.pos_begin);
    ve = min(ve, a.kv.pos_begin + a.shard_count);
    const int T = max(0, ve - vs);
    const int chunk = (T + a.n_split - 1) / a.n_split;
    const int s0 = vs + split * chunk;
    const int s1 = min(ve, s0 + chunk);
    const int64_t row0 = a.kv.row(seq, a.layer, a.kv.pos_begin);
    const int k0 = s0 - a.kv.pos_begin, k1 = s1 - a.kv.pos_begin;
    const int n_tiles = k1 > k0 ? (k1 - k0 + TK - 1) / TK : 0;

    float* alpha_s = reinterpret_cast<float*>(smem);                         // [GH], then m [GH], l [GH]
    float* m_s = alpha_s + kTileGH;
    float* l_s = m_s + kTileGH;
    unsigned char* ring = smem + 128;
    float* part = reinterpret_cast<float*>(ring + (size_t)nst * Ge::STAGE);  // [NC][GH][TK]
    float* p_s = part + NC * kTileGH * TK;                                   // [GH][TK]

    const unsigned char* kg_base = reinterpret_cast<const unsigned char*>(a.kv.k);
    const unsigned char* vg_base = reinterpret_cast<const unsigned char*>(a.kv.v);
    // copies tile `t` of this CTA's keys into ring stage `st` (rows past the end are zero-filled)
    auto issue = [&](int t, int st) {
        unsigned char* ks = ring + (size_t)st * Ge::STAGE;
        unsigned char* vsm = ks + Ge::MAT;
        const int key0 = k0 + t * TK;
        for (int id = tid; id < TK * Ge::GPR; id += kTileThreads) {
            const int key = id / Ge::GPR, col = id - key * Ge::GPR;
            const int tk = key0 + key;
            const int valid = tk < k1;
            const int64_t src = ((row0 + (valid ? tk : k1 - 1)) * a.kv.kv_dim + (int64_t)kvh * D) * EB + col * 16;
            cp_async_16(smem_u32(ks + key * RS + col * 16), kg_base + src, valid ? 16 : 0);
            cp_async_16(smem_u32(vsm + key * RS + col * 16), vg_base + src, valid ? 16 : 0);
        }
        if (NSH > 0) {
            float* ksc = reinterpret_cast<float*>(ks + 2 * Ge::MAT);
            float* vsc = ksc + TK * NSH;
            const int nsr = a.kv.n_scales;
            for (int id = tid; id < TK * NSH; id += kTileThreads) {
                constexpr int NS1 = NSH > 0 ? NSH : 1;  // (the branch is dead when NSH is 0)
                const int key = id / NS1, b = id - key * NS1;
                const int tk = key0 + key;
                const int valid = tk < k1;
                const int64_t si = (row0 + (valid ? tk : k1 - 1)) * nsr + (FMT == KV_Q8_ROW ? 0 : (int64_t)kvh * NSH + b);
                cp_async_4(smem_u32(ksc + id), a.kv.ks + si, valid ? 4 : 0);
                cp_async_4(smem_u32(vsc + id), a.kv.vs + si, valid ? 4 : 0);
            }
        }
    };

    // The first tiles (one per ring stage) do not depend on the query: they are requested before the fused
    // prologue, unless one of them holds the row that the prologue of this (owner) CTA is about to append.
    const bool owner = a.fused.enabled && pos >= s0 && pos < s1;
    const bool first_early = !(owner && (pos - s0) < nst * TK);
    if (first_early) {
        for (int t = 0; t < nst; ++t) {
            if (t < n_tiles) issue(t, t);
            cp_async_commit();
        }
    }
    const float* qsrc = a.q + ((int64_t)item * Hq + (int64_t)kvh * G) * D;
    if (a.fused.enabled) qsrc = fused_rope_prologue(a, item, kvh, seq, pos, owner, smem);
    DECODE_STAMP(1);

    const int c = warp % NC, key_l = (warp / NC) * 32 + lane;  // score phase: slice of the head, key of the tile
    const int dt = tid % DT, kgi = tid / DT;                   // P V phase: 4 bytes of the head, key group

    for (int g0 = 0; g0 < G; g0 += kTileGH) {
        const int gh = min(kTileGH, G - g0);
        const float* qh = qsrc + (int64_t)g0 * D;
        float acc[kTileGH][EPT];
#pragma unroll
        for (int g = 0; g < kTileGH; ++g)
#pragma unroll
            for (int e = 0; e < EPT; ++e) acc[g][e] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f;  // state of head g0 + warp (softmax warps)

        // nst tiles are in flight at any time: one commit group per tile (empty past the end), so the group of
        // tile `it` is complete when at most nst - 1 younger groups are pending
        if (!(g0 == 0 && first_early)) {
            for (int t = 0; t < nst; ++t) {
                if (t < n_tiles) issue(t, t);
                cp_async_commit();
            }
        }
        for (int it = 0; it < n_tiles; ++it) {
            const int st = nst == 1 ? 0 : (it & 1);
            if (nst > 1)
                cp_async_wait<1>();
            else
                cp_async_wait<0>();
            __syncthreads();
            const unsigned char* ks = ring + (size_t)st * Ge::STAGE;
            const unsigned char* vsm = ks + Ge::MAT;
            const float* ksc = reinterpret_cast<const float*>(ks + 2 * Ge::MAT);
            const float* vsc = ksc + TK * NSH;
            const int key0 = k0 + it * TK;

            // ---- scores: this thread's key against slice c of every query head ----
            {
                float dot[kTileGH];
#pragma unroll
                for (int g = 0; g < kTileGH; ++g) dot[g] = 0.0f;
                const unsigned char* kr = ks + key_l * RS + c * CD * EB;
#pragma unroll
                for (int i0 = 0; i0 < CD; i0 += PIECE) {
                    float x[PIECE];
                    const uint4 u = *reinterpret_cast<const uint4*>(kr + i0 * EB);
                    if (FMT == KV_F32) {
                        x[0] = __uint_as_float(u.x); x[1] = __uint_as_float(u.y);
                        x[2] = __uint_as_float(u.z); x[3] = __uint_as_float(u.w);
                    } else if (FMT == KV_BF16) {
                        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            x[2 * i] = __uint_as_float(w4[i] << 16);
                            x[2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
                        }
                    } else {
                        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                        for (int i = 0; i < 16; ++i) x[i] = (float)(signed char)((w4[i >> 2] >> (8 * (i & 3))) & 0xff);
                    }
                    float sc = 1.0f;
                    if (FMT == KV_Q8_BLOCK32) sc = ksc[key_l * NSH + (c * CD + i0) / 32];
#pragma unroll
                    for (int g = 0; g < kTileGH; ++g) {
                        if (g < gh) {
                            const float4* q4 = reinterpret_cast<const float4*>(qh + g * D + c * CD + i0);
                            float pd = 0.0f;
#pragma unroll
                            for (int i = 0; i < PIECE; i += 4) {
                                const float4 qq = q4[i >> 2];
                                pd = fmaf(qq.x, x[i], pd);
                                pd = fmaf(qq.y, x[i + 1], pd);
                                pd = fmaf(qq.z, x[i + 2], pd);
                                pd = fmaf(qq.w, x[i + 3], pd);
                            }
                            dot[g] = FMT == KV_Q8_BLOCK32 ? fmaf(pd, sc, dot[g]) : dot[g] + pd;
                        }
                    }
                }
                float post = a.score_scale;
                if (FMT == KV_Q8_ROW) post *= ksc[key_l];
#pragma unroll
                for (int g = 0; g < kTileGH; ++g)
                    if (g < gh) part[(c * kTileGH + g) * TK + key_l] = dot[g] * post;
            }
            __syncthreads();

            // ---- softmax: warp g owns query head g0 + g ----
            if (warp < gh) {
                float sv[TK / 32];
                float mx = -INFINITY;
#pragma unroll
                for (int r = 0; r < TK / 32; ++r) {
                    const int kk = r * 32 + lane;
                    float s = 0.0f;
#pragma unroll
                    for (int cc = 0; cc < NC; ++cc) s += part[(cc * kTileGH + warp) * TK + kk];
                    sv[r] = key0 + kk < k1 ? s : -INFINITY;
                    mx = fmaxf(mx, sv[r]);
                }
                mx = warp_max(mx);
                const float m_new = fmaxf(m_run, mx);
                const float alpha = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);
                float ps = 0.0f;
#pragma unroll
                for (int r = 0; r < TK / 32; ++r) {
                    const int kk = r * 32 + lane;
                    const float p = m_new == -INFINITY ? 0.0f : exp2f(sv[r] - m_new);
                    ps += p;
                    // the row scale of a q8 value row rides on the probability
                    p_s[warp * TK + kk] = FMT == KV_Q8_ROW ? p * vsc[kk] : p;
                }
                l_run = l_run * alpha + warp_sum(ps);
                m_run = m_new;
                if (lane == 0) alpha_s[warp] = alpha;
            }
            __syncthreads();

            // ---- P V: 4 bytes of the head for the keys of this thread's group ----
            {
#pragma unroll
                for (int g = 0; g < kTileGH; ++g)
                    if (g < gh) {
                        const float al = alpha_s[g];
#pragma unroll
                        for (int e = 0; e < EPT; ++e) acc[g][e] *= al;
                    }
#pragma unroll 4
                for (int kk = kgi * KPG; kk < (kgi + 1) * KPG; ++kk) {
                    const uint32_t u = *reinterpret_cast<const uint32_t*>(vsm + kk * RS + dt * 4);
                    float x[EPT];
                    if (FMT == KV_F32) {
                        x[0] = __uint_as_float(u);
                    } else if (FMT == KV_BF16) {
                        x[0] = __uint_as_float(u << 16);
                        x[EPT - 1] = __uint_as_float(u & 0xffff0000u);
                    } else {
                        float sc = 1.0f;
                        if (FMT == KV_Q8_BLOCK32) sc = vsc[kk * NSH + (dt * 4) / 32];
#pragma unroll
                        for (int e = 0; e < EPT; ++e) x[e] = (float)(signed char)((u >> (8 * e)) & 0xff) * sc;
                    }
#pragma unroll
                    for (int g = 0; g < kTileGH; ++g)
                        if (g < gh) {
                            const float p = p_s[g * TK + kk];
#pragma unroll
                            for (int e = 0; e < EPT; ++e) acc[g][e] = fmaf(p, x[e], acc[g][e]);
                        }
                }
            }
            __syncthreads();  // the stage and the probability arrays are free again
            if (it + nst < n_tiles) issue(it + nst, st);
            cp_async_commit();
        }
        cp_async_wait<0>();
        __syncthreads();
        DECODE_STAMP(2);

        // ---- fold the key groups and store this CTA's state for heads g0 .. g0 + gh ----
        if (warp < gh && lane == 0) {
            m_s[warp] = m_run;
            l_s[warp] = l_run;
        }
        float* red = reinterpret_cast<float*>(ring);  // [KG][gh][D]: ring, partial dots and probabilities are all free now
        if (KG > 1) {
#pragma unroll
            for (int g = 0; g < kTileGH; ++g)
                if (g < gh) {
#pragma unroll
                    for (int e = 0; e < EPT; ++e) red[((size_t)kgi * gh + g) * D + dt * EPT + e] = acc[g][e];
                }
        }
        __syncthreads();
        if (KG > 1) {
            for (int idx = tid; idx < gh * D; idx += kTileThreads) {
                const int g = idx / D, d = idx - g * D;
                float o = 0.0f;
#pragma unroll
                for (int q = 0; q < KG; ++q) o += red[((size_t)q * gh + g) * D + d];
                const int h = kvh * G + g0 + g;
                if (a.n_split == 1) {
                    store_final(a, item, h, d, o, m_s[g], l_s[g]);
                } else {
                    float* pp = a.part + (((int64_t)item * Hq + h) * a.n_split + split) * (D + 2);
                    pp[d] = o;
                    if (d == 0) {
                        pp[D] = m_s[g];
                        pp[D + 1] = l_s[g];
                    }
                }
            }
        } else {
#pragma unroll
            for (int g = 0; g < kTileGH; ++g)
                if (g < gh) {
                    const int h = kvh * G + g0 + g;
#pragma unroll
                    for (int e = 0; e < EPT; ++e) {
                        const int d = dt * EPT + e;
                        if (a.n_split == 1) {
                            store_final(a, item, h, d, acc[g][e], m_s[g], l_s[g]);
                        } else {
                            float* pp = a.part + (((int64_t)item * Hq + h) * a.n_split + split) * (D + 2);
                            pp[d] = acc[g][e];
                            if (d == 0) {
                                pp[D] = m_s[g];
                                pp[D + 1] = l_s[g];
                            }
                        }
                    }
                }
        }
        __syncthreads();  // the ring is free again before the next head group refills it
    }
    DECODE_STAMP(3);
    split_merge_store(a, item, kvh, &s_last, reinterpret_cast<float*>(smem));
    DECODE_STAMP(4);
}

inline bool tile_decode_supported(int fmt, int D) {
    return (fmt == KV_F32 || fmt == KV_BF16 || fmt == KV_Q8_ROW || fmt == KV_Q8_BLOCK32) && (D == 64 || D == 128 || D == 256);
}

struct TilePlan {
    int tk, stage_bytes, nst;
    size_t smem;  // without the fusion scratch and the split-merge weights
    int ctas_per_sm;
};

template <int FMT, int D>
inline TilePlan tile_plan_inst(int nst, int smem_optin) {
    using Ge = TileGeom<FMT, D>;
    TilePlan p{};
    p.tk = Ge::TK;
    p.stage_bytes = Ge::STAGE;
    p.nst = nst;
    p.smem = tile_smem_bytes<FMT, D>(nst);
    const int by_smem = (int)((size_t)(smem_optin + 1024) / (p.smem + 12 * 1024));
    p.ctas_per_sm = by_smem < 1 ? 1 : (by_smem > 4 ? 4 : by_smem);
    return p;
}

template <int FMT>
inline TilePlan tile_plan_fmt(int D, int nst, int smem_optin) {
    switch (D) {
        case 64: return tile_plan_inst<FMT, 64>(nst, smem_optin);
        case 128: return tile_plan_inst<FMT, 128>(nst, smem_optin);
        default: return tile_plan_inst<FMT, 256>(nst, smem_optin);
    }
}

inline TilePlan tile_plan(int fmt, int D, int nst, int smem_optin) {
    switch (fmt) {
        case KV_F32: return tile_plan_fmt<KV_F32>(D, nst, smem_optin);
        case KV_BF16: return tile_plan_fmt<KV_BF16>(D, nst, smem_optin);
        case KV_Q8_ROW: return tile_plan_fmt<KV_Q8_ROW>(D, nst, smem_optin);
        default: return tile_plan_fmt<KV_Q8_BLOCK32>(D, nst, smem_optin);
    }
}

template <int FMT, int D>
inline int launch_tile_inst(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const cudaError_t se = setup.ensure(attn_tile_kernel<FMT, D>, device, smem_optin);
    if (se != cudaSuccess) return (int)se;
    attn_tile_kernel<FMT, D><<<grid, kTileThreads, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

template <int FMT>
inline int launch_tile_fmt(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    switch (a.kv.D) {
        case 64: return launch_tile_inst<FMT, 64>(a, grid, smem, smem_optin, device, stream);
        case 128: return launch_tile_inst<FMT, 128>(a, grid, smem, smem_optin, device, stream);
        case 256: return launch_tile_inst<FMT, 256>(a, grid, smem, smem_optin, device, stream);
        default: return (int)cudaErrorNotSupported;
    }
}

inline int launch_tile_decode(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    switch (a.kv.fmt) {
        case KV_F32: return launch_tile_fmt<KV_F32>(a, grid, smem, smem_optin, device, stream);
        case KV_BF16: return launch_tile_fmt<KV_BF16>(a, grid, smem, smem_optin, device, stream);
        case KV_Q8_ROW: return launch_tile_fmt<KV_Q8_ROW>(a, grid, smem, smem_optin, device, stream);
        case KV_Q8_BLOCK32: return launch_tile_fmt<KV_Q8_BLOCK32>(a, grid, smem, smem_optin, device, stream);
        default: return (int)cudaErrorNotSupported;
    }
}

}  // namespace ggr
