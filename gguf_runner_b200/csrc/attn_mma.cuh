// Split-KV decode over a bf16 cache with the query heads of a KV head packed
// into the M dimension of warp-level tensor-core MMAs (m16n8k16, bf16 -> f32).
//
// Why tensor cores in a bandwidth-bound kernel: with G = n_heads / n_kv_heads
// query heads sharing every cache byte, decode needs 2*G flops per byte of
// bf16 cache; at G = 5..8 the CUDA cores cannot keep up with HBM, the tensor
// cores can with room to spare. Same arithmetic as attention_token
// (src/engine/runtime/inference.rs:1970-2530), online softmax form.
//
// Each warp is an independent split-KV worker: its own cp.async ring of NST
// stages, a stage holding TK = 32 keys of K and V for this KV head in a
// 16-byte-chunk XOR swizzle (chunk ^ (row & 7)) so that ldmatrix is free of
// bank conflicts. The warps of a CTA and then the splits of a (token, kv head)
// are merged exactly as in the CUDA-core kernel.
#pragma once

#include "attn_simt.cuh"
#include "sm100_utils.cuh"

namespace ggr {

constexpr int kMmaTK = 32;
constexpr int kMmaWarps = 4;

struct MmaPlan {
    size_t smem;
    int ctas_per_sm;
    int min_keys;
    int nst;
};

inline bool mma_decode_supported(int D, int G) { return (D == 64 || D == 128) && G >= 1; }

inline MmaPlan mma_plan(int D, int smem_optin) {
    MmaPlan p{};
    const int stage = 2 * kMmaTK * D * 2;
    int nst = 3;
    if ((size_t)kMmaWarps * nst * stage > (size_t)200 * 1024) nst = 2;
    p.nst = nst;
    size_t ring = (size_t)kMmaWarps * nst * stage;
    size_t merge = (size_t)kMmaWarps * 16 * (D + 2) * sizeof(float) + 256;
    p.smem = ring > merge ? ring : merge;
    p.ctas_per_sm = (int)((size_t)(smem_optin + 1024) / (p.smem + 4096));
    if (p.ctas_per_sm < 1) p.ctas_per_sm = 1;
    if (p.ctas_per_sm > 4) p.ctas_per_sm = 4;
    p.min_keys = kMmaWarps * kMmaTK * 2;
    return p;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// copies TK rows of K and V (this KV head's slice) into a swizzled stage
template <int D>
__device__ __forceinline__ void mma_issue_tile(const AttnArgs& a, unsigned char* stage, int64_t row0, int key0,
                                               int key_end, int kvh, int lane) {
    constexpr int rowbytes = D * 2;
    constexpr int cpr = rowbytes / 16;  // 16-byte chunks per row
    constexpr int total = kMmaTK * cpr;
    unsigned char* ks = stage;
    unsigned char* vs = stage + kMmaTK * rowbytes;
    const unsigned char* kg = reinterpret_cast<const unsigned char*>(a.kv.k);
    const unsigned char* vg = reinterpret_cast<const unsigned char*>(a.kv.v);
#pragma unroll 4
    for (int g = lane; g < total; g += 32) {
        const int key = g / cpr, col = g % cpr;
        const int t = key0 + key;
        const int valid = t < key_end;
        const int tc = valid ? t : key_end - 1;
        const int64_t src = ((row0 + tc) * a.kv.kv_dim + (int64_t)kvh * D) * 2 + (int64_t)col * 16;
        const int dst = key * rowbytes + ((col ^ (key & 7)) << 4);
        cp_async_16(smem_u32(ks + dst), kg + src, valid ? 16 : 0);
        cp_async_16(smem_u32(vs + dst), vg + src, valid ? 16 : 0);
    }
}

template <int D, int NST>
__global__ void __launch_bounds__(kMmaWarps * 32) attn_mma_decode_kernel(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;
    constexpr int rowbytes = D * 2;
    constexpr int stage_bytes = 2 * kMmaTK * rowbytes;
    constexpr int KS = D / 16;   // k-steps of Q.K^T
    constexpr int NT = D / 8;    // n-tiles of P.V

    const int G = a.kv.G, Hq = a.kv.Hq;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    // the warp index goes through a broadcast so that the compiler knows everything derived from it (key range,
    // ring addresses, TMA coordinates) is warp-uniform
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int gq = lane >> 2, tq = lane & 3;  // row group and position in the quad

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

    unsigned char* ring = smem + (size_t)warp * NST * stage_bytes;
    const int n_tiles_total = k1 > k0 ? (k1 - k0 + kMmaTK - 1) / kMmaTK : 0;
    const int my_tiles = n_tiles_total > warp ? (n_tiles_total - warp + kMmaWarps - 1) / kMmaWarps : 0;

    for (int g0 = 0; g0 < G; g0 += 16) {
        // Q fragments: rows are query heads g0 + gq and g0 + gq + 8 of this KV head
        uint32_t qf[KS][4];
        {
            const int r0 = g0 + gq, r1 = g0 + gq + 8;
            const float* q0 = a.q + ((int64_t)item * Hq + (int64_t)kvh * G + r0) * D;
            const float* q1 = a.q + ((int64_t)item * Hq + (int64_t)kvh * G + r1) * D;
            const bool v0 = r0 < G, v1 = r1 < G;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int d = ks * 16 + tq * 2;
                float2 x00 = v0 ? *reinterpret_cast<const float2*>(q0 + d) : make_float2(0.f, 0.f);
                float2 x01 = v0 ? *reinterpret_cast<const float2*>(q0 + d + 8) : make_float2(0.f, 0.f);
                float2 x10 = v1 ? *reinterpret_cast<const float2*>(q1 + d) : make_float2(0.f, 0.f);
                float2 x11 = v1 ? *reinterpret_cast<const float2*>(q1 + d + 8) : make_float2(0.f, 0.f);
                qf[ks][0] = pack_bf16x2(x00.x * a.score_scale, x00.y * a.score_scale);
                qf[ks][1] = pack_bf16x2(x10.x * a.score_scale, x10.y * a.score_scale);
                qf[ks][2] = pack_bf16x2(x01.x * a.score_scale, x01.y * a.score_scale);
                qf[ks][3] = pack_bf16x2(x11.x * a.score_scale, x11.y * a.score_scale);
            }
        }
        float o[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
        for (int s = 0; s < NST - 1; ++s) {
            if (s < my_tiles)
                mma_issue_tile<D>(a, ring + (size_t)s * stage_bytes, row0, k0 + (warp + s * kMmaWarps) * kMmaTK, k1, kvh,
                                  lane);
            cp_async_commit();
        }

        for (int it = 0; it < my_tiles; ++it) {
            cp_async_wait<NST - 2>();
            __syncwarp();
            const uint32_t kt = smem_u32(ring + (size_t)(it % NST) * stage_bytes);
            const uint32_t vt = kt + kMmaTK * rowbytes;
            const int key0 = k0 + (warp + it * kMmaWarps) * kMmaTK;

            // S = Q K^T for 32 keys: 4 n-tiles of 8 keys
            float sc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {  // pairs of n-tiles
                    const int row = jp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
                    const int chunkc = 2 * ks + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(kt + row * rowbytes + ((chunkc ^ (row & 7)) << 4), b0, b1, b2, b3);
                    mma_bf16_16816(sc[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma_bf16_16816(sc[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
                }
            }
            // mask keys past the end of this CTA's range
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kb = key0 + j * 8 + tq * 2;
                if (kb >= k1) sc[j][0] = sc[j][2] = -INFINITY;
                if (kb + 1 >= k1) sc[j][1] = sc[j][3] = -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // every tile holds at least one valid key, so the new maxima are finite
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
            uint32_t pf[2][4];  // P as A fragments for the two 16-key k-steps
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p0 = exp2f(sc[j][0] - mn0), p1 = exp2f(sc[j][1] - mn0);
                const float p2 = exp2f(sc[j][2] - mn1), p3 = exp2f(sc[j][3] - mn1);
                ps0 += p0 + p1;
                ps1 += p2 + p3;
                pf[j >> 1][(j & 1) * 2] = pack_bf16x2(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16x2(p2, p3);
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                o[nt][0] *= al0;
                o[nt][1] *= al0;
                o[nt][2] *= al1;
                o[nt][3] *= al1;
            }
            // O += P V: k-steps of 16 keys, n-tiles of 8 head elements (two per ldmatrix)
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int chunkc = 2 * np + ((lane >> 4) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vt + row * rowbytes + ((chunkc ^ (row & 7)) << 4), b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
                    mma_bf16_16816(o[2 * np + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
                }
            }
            __syncwarp();
            const int nt_ = it + NST - 1;
            if (nt_ < my_tiles)
                mma_issue_tile<D>(a, ring + (size_t)(nt_ % NST) * stage_bytes, row0,
                                  k0 + (warp + nt_ * kMmaWarps) * kMmaTK, k1, kvh, lane);
            cp_async_commit();
        }
        cp_async_wait<0>();

        // row sums live spread over the quad
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

        __syncthreads();  // all rings drained: reuse shared memory as the merge area
        float* wacc = reinterpret_cast<float*>(smem);  // [W][16][D]
        float* wm = wacc + kMmaWarps * 16 * D;          // [W][16]
        float* wl = wm + kMmaWarps * 16;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int d = nt * 8 + tq * 2;
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq) * D + d]) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq + 8) * D + d]) = make_float2(o[nt][2], o[nt][3]);
        }
        if (tq == 0) {
            wm[warp * 16 + gq] = m0;
            wm[warp * 16 + gq + 8] = m1;
            wl[warp * 16 + gq] = l0;
            wl[warp * 16 + gq + 8] = l1;
        }
        __syncthreads();
        cta_merge_store(a, wacc, wm, wl, kMmaWarps, 16, g0, min(16, G - g0), item, kvh, split);
        __syncthreads();
    }
    split_merge_store(a, item, kvh, &s_last, reinterpret_cast<float*>(smem));
}

template <int D, int NST>
inline int launch_mma_inst(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const cudaError_t se = setup.ensure(attn_mma_decode_kernel<D, NST>, device, smem_optin);
    if (se != cudaSuccess) return (int)se;
    attn_mma_decode_kernel<D, NST><<<grid, kMmaWarps * 32, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

inline int launch_mma_decode(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device,
                             cudaStream_t stream) {
    switch (a.kv.D) {
        case 64: return launch_mma_inst<64, 3>(a, grid, smem, smem_optin, device, stream);
        case 128: return launch_mma_inst<128, 3>(a, grid, smem, smem_optin, device, stream);
        default: return (int)cudaErrorNotSupported;
    }
}

// ---- TMA-fed variant ---------------------------------------------------------------------------
// Same arithmetic, different data movement and occupancy: eight warps per CTA (two per scheduler, so
// one warp's MMA / ldmatrix latencies hide behind the other's), each warp with its own ring of NST
// stages of 16 keys that one lane fills with four bulk tensor copies (two 64-column boxes of K, two
// of V, 128-byte swizzle) completing on a per-stage mbarrier, instead of 512 cp.async per lane-set.
// The running output is rescaled only when a row maximum grows by more than 2^8.

constexpr int kTmaTK = 16;
constexpr int kTmaWarps = 8;
constexpr int kTmaNST = 3;

inline bool mma_tma_decode_supported(int D) { return D == 64 || D == 128; }

inline MmaPlan mma_tma_plan(int D, int smem_optin) {
    MmaPlan p{};
    const int stage = 2 * kTmaTK * D * 2;
    p.nst = kTmaNST;
    size_t ring = (size_t)kTmaWarps * kTmaNST * stage;
    size_t merge = (size_t)kTmaWarps * 16 * (D + 8 + 2) * sizeof(float) + 256;
    p.smem = (ring > merge ? ring : merge) + 1024;  // slack to align the ring to the swizzle atom
    p.ctas_per_sm = (int)((size_t)(smem_optin + 1024) / (p.smem + 4096));
    if (p.ctas_per_sm < 1) p.ctas_per_sm = 1;
    if (p.ctas_per_sm > 4) p.ctas_per_sm = 4;
    p.min_keys = kTmaWarps * kTmaTK * 2;
    return p;
}

template <int D>
__global__ void __launch_bounds__(kTmaWarps * 32) attn_mma_tma_decode_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                             const __grid_constant__ CUtensorMap tmV,
                                                                             AttnArgs a) {
    using namespace tc;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(8) uint64_t s_full[kTmaWarps][kTmaNST];
    __shared__ int s_last;
    __shared__ int s_abort;
    constexpr int NBLK = D / 64;                   // 64-column (128-byte) blocks of a row
    constexpr uint32_t BLK_BYTES = kTmaTK * 128;   // [16 rows][128 bytes]
    constexpr uint32_t MAT_BYTES = NBLK * BLK_BYTES;
    constexpr uint32_t STAGE_BYTES = 2 * MAT_BYTES;
    constexpr int KS = D / 16;
    constexpr int NT = D / 8;
    constexpr int NST = kTmaNST;

    const int G = a.kv.G, Hq = a.kv.Hq;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    // the warp index goes through a broadcast so that the compiler knows everything derived from it (key range,
    // ring addresses, TMA coordinates) is warp-uniform
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int gq = lane >> 2, tq = lane & 3;
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

    const uint32_t ring_base = (smem_u32(smem) + 1023u) & ~1023u;
    unsigned char* smem_al = smem + (ring_base - smem_u32(smem));
    const uint32_t ring = ring_base + (uint32_t)warp * NST * STAGE_BYTES;
    const int n_tiles_total = k1 > k0 ? (k1 - k0 + kTmaTK - 1) / kTmaTK : 0;
    const int my_tiles = n_tiles_total > warp ? (n_tiles_total - warp + kTmaWarps - 1) / kTmaWarps : 0;

    DECODE_STAMP(0);
    if (tid == 0) s_abort = 0;
    if (lane == 0) {
        for (int s = 0; s < NST; ++s) mbar_init(smem_u32(&s_full[warp][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int* abortp = &s_abort;

    auto issue = [&](int tile_idx, int stage) {
        // one lane: K and V rows [key, key + 16) of this KV head, 64 columns per box
        const uint32_t bar = smem_u32(&s_full[warp][stage]);
        const uint32_t dst = ring + (uint32_t)stage * STAGE_BYTES;
        const int y = (int)(row0 + k0 + (int64_t)(warp + tile_idx * kTmaWarps) * kTmaTK);
        mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
        for (int b = 0; b < NBLK; ++b) {
            tma_load_2d(dst + b * BLK_BYTES, &tmK, kvh * D + b * 64, y, bar);
            tma_load_2d(dst + MAT_BYTES + b * BLK_BYTES, &tmV, kvh * D + b * 64, y, bar);
        }
    };

    // The first tiles are requested before the fused prologue (they do not depend on the query), so the
    // rotation of q and the append hide behind their latency. The one exception is the warp of the owner CTA
    // whose first tiles would hold the row that the prologue is about to append.
    const bool owner = a.fused.enabled && pos >= s0 && pos < s1;
    bool prefetched = true;
    if (owner) {
        const int tile_pos = (pos - s0) / kTmaTK;
        if (tile_pos % kTmaWarps == warp && tile_pos / kTmaWarps < NST - 1) prefetched = false;
    }
    if (prefetched && lane == 0) {
        for (int s = 0; s < NST - 1 && s < my_tiles; ++s) issue(s, s);
    }
    const float* qsrc = a.q + ((int64_t)item * Hq + (int64_t)kvh * G) * D;
    if (a.fused.enabled) qsrc = fused_rope_prologue(a, item, kvh, seq, pos, owner, smem);
    DECODE_STAMP(1);

    uint32_t use_count = 0;  // tiles consumed so far by this warp over all head groups (barrier phases)
    for (int g0 = 0; g0 < G; g0 += 16) {
        uint32_t qf[KS][4];
        {
            const int r0 = g0 + gq, r1 = g0 + gq + 8;
            const float* q0 = qsrc + (int64_t)r0 * D;
            const float* q1 = qsrc + (int64_t)r1 * D;
            const bool v0 = r0 < G, v1 = r1 < G;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int d = ks * 16 + tq * 2;
                float2 x00 = v0 ? *reinterpret_cast<const float2*>(q0 + d) : make_float2(0.f, 0.f);
                float2 x01 = v0 ? *reinterpret_cast<const float2*>(q0 + d + 8) : make_float2(0.f, 0.f);
                float2 x10 = v1 ? *reinterpret_cast<const float2*>(q1 + d) : make_float2(0.f, 0.f);
                float2 x11 = v1 ? *reinterpret_cast<const float2*>(q1 + d + 8) : make_float2(0.f, 0.f);
                qf[ks][0] = pack_bf16x2(x00.x * a.score_scale, x00.y * a.score_scale);
                qf[ks][1] = pack_bf16x2(x10.x * a.score_scale, x10.y * a.score_scale);
                qf[ks][2] = pack_bf16x2(x01.x * a.score_scale, x01.y * a.score_scale);
                qf[ks][3] = pack_bf16x2(x11.x * a.score_scale, x11.y * a.score_scale);
            }
        }
        float o[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        if (lane == 0 && !(g0 == 0 && prefetched)) {
            for (int s = 0; s < NST - 1 && s < my_tiles; ++s) issue(s, (int)((use_count + s) % NST));
        }
        bool ok = true;
        for (int it = 0; it < my_tiles; ++it) {
            const uint32_t u = use_count + it;
            const int stage = (int)(u % NST);
            ok = mbar_wait(smem_u32(&s_full[warp][stage]), (u / NST) & 1u, abortp);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t kt = ring + (uint32_t)stage * STAGE_BYTES;
            const uint32_t vt = kt + MAT_BYTES;
            const int key0 = k0 + (warp + it * kTmaWarps) * kTmaTK;

            // S = Q K^T for 16 keys: 2 n-tiles of 8 keys
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.f;
            sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int row = (lane & 7) + ((lane >> 4) & 1) * 8;
                const int chunkc = 2 * ks + ((lane >> 3) & 1);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kt + (chunkc >> 3) * BLK_BYTES + row * 128 + (((chunkc & 7) ^ (row & 7)) << 4), b0, b1, b2, b3);
                mma_bf16_16816(sc[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_bf16_16816(sc[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int kb = key0 + j * 8 + tq * 2;
                if (kb >= k1) sc[j][0] = sc[j][2] = -INFINITY;
                if (kb + 1 >= k1) sc[j][1] = sc[j][3] = -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // lazy rescale: move the reference maximum only when it grows by more than 8 (log2 units)
            const bool need0 = mx0 > m0 + 8.0f, need1 = mx1 > m1 + 8.0f;
            if (__any_sync(0xffffffffu, need0 || need1)) {
                const float al0 = need0 ? exp2f(m0 - mx0) : 1.0f;
                const float al1 = need1 ? exp2f(m1 - mx1) : 1.0f;
                if (need0) m0 = mx0;
                if (need1) m1 = mx1;
                l0 *= al0;
                l1 *= al1;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[nt][0] *= al0;
                    o[nt][1] *= al0;
                    o[nt][2] *= al1;
                    o[nt][3] *= al1;
                }
            }
            uint32_t pf[4];
            {
                const float p00 = exp2f(sc[0][0] - m0), p01 = exp2f(sc[0][1] - m0);
                const float p02 = exp2f(sc[0][2] - m1), p03 = exp2f(sc[0][3] - m1);
                const float p10 = exp2f(sc[1][0] - m0), p11 = exp2f(sc[1][1] - m0);
                const float p12 = exp2f(sc[1][2] - m1), p13 = exp2f(sc[1][3] - m1);
                l0 += (p00 + p01) + (p10 + p11);
                l1 += (p02 + p03) + (p12 + p13);
                pf[0] = pack_bf16x2(p00, p01);
                pf[1] = pack_bf16x2(p02, p03);
                pf[2] = pack_bf16x2(p10, p11);
                pf[3] = pack_bf16x2(p12, p13);
            }
            // O += P V: one k-step of 16 keys, n-tiles of 8 head elements (two per ldmatrix)
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunkc = 2 * np + ((lane >> 4) & 1);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vt + (chunkc >> 3) * BLK_BYTES + row * 128 + (((chunkc & 7) ^ (row & 7)) << 4), b0, b1, b2,
                                  b3);
                mma_bf16_16816(o[2 * np], pf[0], pf[1], pf[2], pf[3], b0, b1);
                mma_bf16_16816(o[2 * np + 1], pf[0], pf[1], pf[2], pf[3], b2, b3);
            }
            __syncwarp();
            const int nt_ = it + NST - 1;
            if (lane == 0 && nt_ < my_tiles) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(nt_, (int)((use_count + nt_) % NST));
            }
        }
        use_count += my_tiles;

        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

        if (s_abort) {
            for (int i = 0; i < 500; ++i) __nanosleep(1000);  // let copies in flight land
        }
        __syncthreads();  // all rings drained: reuse shared memory as the merge area
        DECODE_STAMP(2);
        // rows are padded by 8 floats: the eight row groups of a warp then hit different banks
        constexpr int LD = D + 8;
        float* wacc = reinterpret_cast<float*>(smem_al);  // [W][16][LD]
        float* wm = wacc + kTmaWarps * 16 * LD;
        float* wl = wm + kTmaWarps * 16;
        const bool row0_used = g0 + gq < G, row1_used = g0 + gq + 8 < G;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int d = nt * 8 + tq * 2;
            if (row0_used) *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq) * LD + d]) = make_float2(o[nt][0], o[nt][1]);
            if (row1_used) *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq + 8) * LD + d]) = make_float2(o[nt][2], o[nt][3]);
        }
        if (tq == 0) {
            wm[warp * 16 + gq] = m0;
            wm[warp * 16 + gq + 8] = m1;
            wl[warp * 16 + gq] = l0;
            wl[warp * 16 + gq + 8] = l1;
        }
        __syncthreads();
        cta_merge_store(a, wacc, wm, wl, kTmaWarps, 16, g0, min(16, G - g0), item, kvh, split, LD);
        __syncthreads();
    }
    if (tid == 0 && s_abort && a.err) atomicExch(a.err, 1);
    DECODE_STAMP(3);
    split_merge_store(a, item, kvh, &s_last, reinterpret_cast<float*>(smem_al));
    DECODE_STAMP(4);
}

template <int D>
inline int launch_mma_tma_inst(const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a, dim3 grid, size_t smem,
                               int smem_optin, int device, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const cudaError_t se = setup.ensure(attn_mma_tma_decode_kernel<D>, device, smem_optin);
    if (se != cudaSuccess) return (int)se;
    attn_mma_tma_decode_kernel<D><<<grid, kTmaWarps * 32, smem, stream>>>(tk, tv, a);
    return (int)cudaGetLastError();
}

// tk / tv: tensor maps over the whole K and V arrays with a box of 64 columns x 16 rows
inline int launch_mma_tma_decode(const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a, dim3 grid, size_t smem,
                                 int smem_optin, int device, cudaStream_t stream) {
    switch (a.kv.D) {
        case 64: return launch_mma_tma_inst<64>(tk, tv, a, grid, smem, smem_optin, device, stream);
        case 128: return launch_mma_tma_inst<128>(tk, tv, a, grid, smem, smem_optin, device, stream);
        default: return (int)cudaErrorNotSupported;
    }
}

}  // namespace ggr
