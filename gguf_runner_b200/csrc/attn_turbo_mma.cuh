// Split-KV decode over a TurboQuant cache on the tensor cores (head_dim 128, up to 16 query heads per KV head).
//
// The CUDA-core kernel (attn_turbo.cuh) spends about 4 * G * D lane operations per key. Here a key costs a few
// table lookups: every warp expands its 16-key tile of packed codes into four bf16 tiles in shared memory,
//   C_k, C_v : centroid of the 2-bit code          S_k, S_v : +1 / -1 of the residual sign bit
// and the query heads of the KV head ride in the M dimension of m16n8k16 MMAs, as in attn_mma.cuh:
//   score = sigma_k * (Q_r C_k^T) + rho_k * (Q_p S_k^T)          (src/engine/runtime/inference.rs:1246-1269)
//   O_base += (p * sigma_v) C_v,   O_res += (p * rho_v) S_v      (:1284-1306)
// sigma and rho are applied in f32 (to the scores) or folded into P (for the values), so the only roundings beyond
// the reference's arithmetic are bf16 q, bf16 centroids and bf16 P: the bf16-cache tolerance class.
// The inverse transforms (:1323-1334) run once per CTA on the merged accumulators; the result joins the common
// split merge.
//
// Per warp: a 3-stage cp.async ring of raw tiles (16 keys: 512 B codes + 256 B sign bits for K and for V, and
// four floats per key) and one set of expanded tiles (4 x 4 KB, rows swizzled by 16-byte chunk ^ (row & 7)).
#pragma once

#include "attn_mma.cuh"
#include "attn_turbo.cuh"

namespace ggr {

constexpr int kTmWarps = 8;
constexpr int kTmTK = 16;
constexpr int kTmNST = 3;
constexpr int kTmD = 128;
constexpr int kTmRawBytes = 2 * (kTmTK * kTmD / 4) + 2 * (kTmTK * kTmD / 8) + 4 * kTmTK * 4;  // 1792
constexpr int kTmTileBytes = kTmTK * kTmD * 2;                                                  // 4096
constexpr int kTmWarpBytes = kTmNST * kTmRawBytes + 4 * kTmTileBytes;                          // 21760
constexpr int kTmLD = 2 * kTmD + 8;  // merge rows: base | residual accumulators, padded against bank conflicts

inline bool turbo_mma_supported(int D, int G) { return D == kTmD && G <= 16; }

// byte offset of the query preparation area (q_r, q_p: 2 x 16 x D floats) behind the work area, whose three uses
// (rings and tiles; warp merge; split merge weights) follow one another
inline size_t turbo_mma_prep_offset(int G, int n_split) {
    const size_t work = (size_t)kTmWarps * kTmWarpBytes;
    const size_t merge = ((size_t)kTmWarps * 16 * kTmLD + 2 * kTmWarps * 16 + 96 + (size_t)16 * 2 * kTmD) * 4;
    const size_t split = n_split > 1 ? ((size_t)2 * G * n_split + 2 * G + split_merge_sub_floats(G, kTmD)) * 4 : 0;
    size_t m = work > merge ? work : merge;
    if (split > m) m = split;
    return (m + 127) & ~(size_t)127;
}
inline size_t turbo_mma_smem_bytes(int G, int n_split) { return turbo_mma_prep_offset(G, n_split) + (size_t)2 * 16 * kTmD * 4; }

// one 16-key raw tile of this warp: codes and sign bits of K and V, sigma and residual norm
__device__ __forceinline__ void turbo_mma_issue(const AttnArgs& a, unsigned char* raw, int64_t row0, int key0, int key_end,
                                                int kvh, int lane) {
    constexpr int D = kTmD;
    const int kv_dim = a.kv.kv_dim, Hkv = a.kv.Hkv;
    unsigned char* kc = raw;
    unsigned char* vc = kc + kTmTK * D / 4;
    unsigned char* ksg = vc + kTmTK * D / 4;
    unsigned char* vsg = ksg + kTmTK * D / 8;
    float* scal = reinterpret_cast<float*>(vsg + kTmTK * D / 8);  // [4][16]: sigma_k, gamma_k, sigma_v, gamma_v
    {
        const int key = lane >> 1, c = lane & 1, t = key0 + key;
        const int valid = t < key_end, tc = valid ? t : key_end - 1;
        const int64_t eo = (row0 + tc) * kv_dim + (int64_t)kvh * D;
        cp_async_16(smem_u32(kc + key * 32 + c * 16), reinterpret_cast<const unsigned char*>(a.kv.k) + eo / 4 + c * 16, valid ? 16 : 0);
        cp_async_16(smem_u32(vc + key * 32 + c * 16), reinterpret_cast<const unsigned char*>(a.kv.v) + eo / 4 + c * 16, valid ? 16 : 0);
    }
    {
        const int key = lane & 15, t = key0 + key;
        const int valid = t < key_end, tc = valid ? t : key_end - 1;
        const int64_t eo = (row0 + tc) * kv_dim + (int64_t)kvh * D, aux = (row0 + tc) * Hkv + kvh;
        if (lane < 16) {
            cp_async_16(smem_u32(ksg + key * 16), a.kv.k_sign + eo / 8, valid ? 16 : 0);
            cp_async_4(smem_u32(scal + key), a.kv.ks + aux, valid ? 4 : 0);
            cp_async_4(smem_u32(scal + 16 + key), a.kv.k_rn + aux, valid ? 4 : 0);
        } else {
            cp_async_16(smem_u32(vsg + key * 16), a.kv.v_sign + eo / 8, valid ? 16 : 0);
            cp_async_4(smem_u32(scal + 32 + key), a.kv.vs + aux, valid ? 4 : 0);
            cp_async_4(smem_u32(scal + 48 + key), a.kv.v_rn + aux, valid ? 4 : 0);
        }
    }
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Eight 2-bit codes (16 bits) -> eight bf16 centroids (four words). The codes are first spread into the eight
// nibbles of a word; four nibbles at a time then select the high and the low bytes of
// bf16(-1.510417, -0.45278, 0.45278, 1.510417) = 0xBFC1, 0xBEE8, 0x3EE8, 0x3FC1 from two table registers, and two
// more permutes interleave them.
__device__ __forceinline__ uint4 turbo_centroids8(uint32_t w) {
    uint32_t x = w;
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    const uint32_t hi_tab = 0x3F3EBEBFu, lo_tab = 0xC1E8E8C1u;
    const uint32_t s0 = x & 0xFFFFu, s1 = x >> 16;
    const uint32_t hi0 = prmt(hi_tab, lo_tab, s0), lo0 = prmt(hi_tab, lo_tab, s0 | 0x4444u);
    const uint32_t hi1 = prmt(hi_tab, lo_tab, s1), lo1 = prmt(hi_tab, lo_tab, s1 | 0x4444u);
    return make_uint4(prmt(lo0, hi0, 0x5140u), prmt(lo0, hi0, 0x7362u), prmt(lo1, hi1, 0x5140u), prmt(lo1, hi1, 0x7362u));
}

// Eight sign bits (1 = positive) -> eight bf16 values +1 / -1: bits spread into nibbles select 0xBF or 0x3F as
// the high byte, the low byte is 0x80.
__device__ __forceinline__ uint4 turbo_signs8(uint32_t sb) {
    uint32_t x = sb;
    x = (x | (x << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    x = (x | (x << 3)) & 0x11111111u;
    const uint32_t h0 = prmt(0x00003FBFu, 0u, x & 0xFFFFu), h1 = prmt(0x00003FBFu, 0u, x >> 16);
    const uint32_t c80 = 0x80808080u;
    return make_uint4(prmt(h0, c80, 0x1404u), prmt(h0, c80, 0x3424u), prmt(h1, c80, 0x1404u), prmt(h1, c80, 0x3424u));
}

// expands 64 codes (16 bytes) and 64 sign bits (8 bytes) of one key half into bf16 chunks of the two tiles;
// shared memory only sees the 16-byte stores (the lookups are register arithmetic)
__device__ __forceinline__ void turbo_mma_expand(const unsigned char* codes, const unsigned char* signs, unsigned char* ctile,
                                                 unsigned char* stile, int key, int half) {
    const uint4 cw = *reinterpret_cast<const uint4*>(codes);
    const uint2 sw = *reinterpret_cast<const uint2*>(signs);
    const uint32_t cwords[4] = {cw.x, cw.y, cw.z, cw.w};
    const uint32_t swords[2] = {sw.x, sw.y};
    const int row_off = key * (kTmD * 2), sw7 = key & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // chunk j: elements half * 64 + 8 j .. + 7
        const uint32_t w = (cwords[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        const uint32_t sb = (swords[j >> 2] >> ((j & 3) * 8)) & 0xffu;
        const int off = row_off + (((half * 8 + j) ^ sw7) << 4);
        *reinterpret_cast<uint4*>(ctile + off) = turbo_centroids8(w);
        *reinterpret_cast<uint4*>(stile + off) = turbo_signs8(sb);
    }
}

__global__ void __launch_bounds__(kTmWarps * 32) attn_turbo_mma_kernel(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char tsm8[];
    __shared__ int s_last;
    constexpr int D = kTmD, KS = D / 16, NT = D / 8, rowbytes = D * 2;
    const int G = a.kv.G, Hq = a.kv.Hq;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int gq = lane >> 2, tq = lane & 3;

    int seq, pos;
    a.items.get(item, seq, pos);
    int vs, ve;
    a.vis.range(pos, vs, ve);
    vs = max(vs, a.kv.pos_begin);
    ve = min(ve, a.kv.pos_begin + a.shard_count);
    const int T = max(0, ve - vs);
    const int chunk = (T + a.n_split - 1) / a.n_split;
    const int s0 = vs + split * chunk, s1 = min(ve, s0 + chunk);
    const int64_t row0 = a.kv.row(seq, a.layer, a.kv.pos_begin);
    const int k0 = s0 - a.kv.pos_begin, k1 = s1 - a.kv.pos_begin;
    const int n_tiles_total = k1 > k0 ? (k1 - k0 + kTmTK - 1) / kTmTK : 0;
    const int my_tiles = n_tiles_total > warp ? (n_tiles_total - warp + kTmWarps - 1) / kTmWarps : 0;

    unsigned char* wbase = tsm8 + (size_t)warp * kTmWarpBytes;
    unsigned char* tiles = wbase + kTmNST * kTmRawBytes;  // C_k, S_k, C_v, S_v
    float* qr = reinterpret_cast<float*>(tsm8 + a.stage_bytes);  // [16][D], behind the work area (offset set by the host)
    float* qp = qr + 16 * D;

    // the first raw tiles are requested before the query preparation
    auto issue = [&](int tile_idx) {
        if (tile_idx < my_tiles)
            turbo_mma_issue(a, wbase + (size_t)(tile_idx % kTmNST) * kTmRawBytes, row0,
                            k0 + (warp + tile_idx * kTmWarps) * kTmTK, k1, kvh, lane);
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kTmNST - 1; ++s) issue(s);

    // query preparation (:954-968): q_r = T(q; rot_pre, rot_post), q_p = T(q_r; res_pre, res_post)
    const unsigned char* rot_pre = turbo_sign_slot(a.kv, 0, a.layer, kvh);
    const unsigned char* rot_post = turbo_sign_slot(a.kv, 1, a.layer, kvh);
    const unsigned char* res_pre = turbo_sign_slot(a.kv, 2, a.layer, kvh);
    const unsigned char* res_post = turbo_sign_slot(a.kv, 3, a.layer, kvh);
    const float* qsrc = a.q + ((int64_t)item * Hq + (int64_t)kvh * G) * D;
    for (int g = warp; g < 16; g += kTmWarps) {
        for (int i = lane; i < D; i += 32) qr[g * D + i] = g < G ? qsrc[(int64_t)g * D + i] : 0.0f;
        __syncwarp();
        if (g < G) turbo_transform_warp(qr + g * D, D, rot_pre, rot_post, lane);
        for (int i = lane; i < D; i += 32) qp[g * D + i] = qr[g * D + i];
        __syncwarp();
        if (g < G) turbo_transform_warp(qp + g * D, D, res_pre, res_post, lane);
    }
    __syncthreads();

    // A fragments of Q_r and Q_p: rows gq and gq + 8, scores come out in log2 units
    uint32_t qfr[KS][4], qfp[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int d = ks * 16 + tq * 2;
        const float sc_ = a.score_scale;
        qfr[ks][0] = pack_bf16x2(qr[gq * D + d] * sc_, qr[gq * D + d + 1] * sc_);
        qfr[ks][1] = pack_bf16x2(qr[(gq + 8) * D + d] * sc_, qr[(gq + 8) * D + d + 1] * sc_);
        qfr[ks][2] = pack_bf16x2(qr[gq * D + d + 8] * sc_, qr[gq * D + d + 9] * sc_);
        qfr[ks][3] = pack_bf16x2(qr[(gq + 8) * D + d + 8] * sc_, qr[(gq + 8) * D + d + 9] * sc_);
        qfp[ks][0] = pack_bf16x2(qp[gq * D + d] * sc_, qp[gq * D + d + 1] * sc_);
        qfp[ks][1] = pack_bf16x2(qp[(gq + 8) * D + d] * sc_, qp[(gq + 8) * D + d + 1] * sc_);
        qfp[ks][2] = pack_bf16x2(qp[gq * D + d + 8] * sc_, qp[gq * D + d + 9] * sc_);
        qfp[ks][3] = pack_bf16x2(qp[(gq + 8) * D + d + 8] * sc_, qp[(gq + 8) * D + d + 9] * sc_);
    }
    const float rho_unit = __fsqrt_rn(__fdiv_rn(1.57079632679489661923f, (float)D));  // :975-982

    float ob[NT][4], orr[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        ob[nt][0] = ob[nt][1] = ob[nt][2] = ob[nt][3] = 0.f;
        orr[nt][0] = orr[nt][1] = orr[nt][2] = orr[nt][3] = 0.f;
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const uint32_t t_ck = smem_u32(tiles), t_sk = t_ck + kTmTileBytes, t_cv = t_sk + kTmTileBytes, t_sv = t_cv + kTmTileBytes;
    for (int it = 0; it < my_tiles; ++it) {
        cp_async_wait<kTmNST - 2>();
        __syncwarp();
        const unsigned char* raw = wbase + (size_t)(it % kTmNST) * kTmRawBytes;
        const float* scal = reinterpret_cast<const float*>(raw + 2 * (kTmTK * D / 4) + 2 * (kTmTK * D / 8));
        const int key0 = k0 + (warp + it * kTmWarps) * kTmTK;
        {
            // eight consecutive lanes expand eight different keys: their 16-byte stores then fall into different banks
            const int key = lane & 15, half = lane >> 4;
            turbo_mma_expand(raw + key * 32 + half * 16, raw + 2 * (kTmTK * D / 4) + key * 16 + half * 8, tiles,
                             tiles + kTmTileBytes, key, half);
            turbo_mma_expand(raw + kTmTK * D / 4 + key * 32 + half * 16,
                             raw + 2 * (kTmTK * D / 4) + kTmTK * D / 8 + key * 16 + half * 8, tiles + 2 * kTmTileBytes,
                             tiles + 3 * kTmTileBytes, key, half);
        }
        __syncwarp();

        // base and residual scores of 16 keys: 2 n-tiles of 8 keys each
        float sb[2][4], sr[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sb[j][0] = sb[j][1] = sb[j][2] = sb[j][3] = sr[j][0] = sr[j][1] = sr[j][2] = sr[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int row = (lane & 7) + ((lane >> 4) & 1) * 8;
            const int chunkc = 2 * ks + ((lane >> 3) & 1);
            const uint32_t off = row * rowbytes + ((chunkc ^ (row & 7)) << 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(t_ck + off, b0, b1, b2, b3);
            mma_bf16_16816(sb[0], qfr[ks][0], qfr[ks][1], qfr[ks][2], qfr[ks][3], b0, b1);
            mma_bf16_16816(sb[1], qfr[ks][0], qfr[ks][1], qfr[ks][2], qfr[ks][3], b2, b3);
            ldmatrix_x4(t_sk + off, b0, b1, b2, b3);
            mma_bf16_16816(sr[0], qfp[ks][0], qfp[ks][1], qfp[ks][2], qfp[ks][3], b0, b1);
            mma_bf16_16816(sr[1], qfp[ks][0], qfp[ks][1], qfp[ks][2], qfp[ks][3], b2, b3);
        }
        float sc[2][4], vsig[2][2], vrho[2][2];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int kk = j * 8 + tq * 2 + i;
                const float sig = scal[kk], rho = scal[16 + kk] * rho_unit;
                vsig[j][i] = scal[32 + kk];
                vrho[j][i] = scal[48 + kk] * rho_unit;
                const bool in = key0 + kk < k1;
                sc[j][i] = in ? fmaf(sig, sb[j][i], rho * sr[j][i]) : -INFINITY;
                sc[j][2 + i] = in ? fmaf(sig, sb[j][2 + i], rho * sr[j][2 + i]) : -INFINITY;
            }
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
            const float al0 = need0 ? exp2f(m0 - mx0) : 1.0f, al1 = need1 ? exp2f(m1 - mx1) : 1.0f;
            if (need0) m0 = mx0;
            if (need1) m1 = mx1;
            l0 *= al0;
            l1 *= al1;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                ob[nt][0] *= al0; ob[nt][1] *= al0; ob[nt][2] *= al1; ob[nt][3] *= al1;
                orr[nt][0] *= al0; orr[nt][1] *= al0; orr[nt][2] *= al1; orr[nt][3] *= al1;
            }
        }
        uint32_t pfb[4], pfr[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float p0 = exp2f(sc[j][0] - m0), p1 = exp2f(sc[j][1] - m0);
            const float p2 = exp2f(sc[j][2] - m1), p3 = exp2f(sc[j][3] - m1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            pfb[2 * j] = pack_bf16x2(p0 * vsig[j][0], p1 * vsig[j][1]);
            pfb[2 * j + 1] = pack_bf16x2(p2 * vsig[j][0], p3 * vsig[j][1]);
            pfr[2 * j] = pack_bf16x2(p0 * vrho[j][0], p1 * vrho[j][1]);
            pfr[2 * j + 1] = pack_bf16x2(p2 * vrho[j][0], p3 * vrho[j][1]);
        }
        // O_base += P_base C_v, O_res += P_res S_v: one k-step of 16 keys, two n-tiles per ldmatrix
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
            const int chunkc = 2 * np + ((lane >> 4) & 1);
            const uint32_t off = row * rowbytes + ((chunkc ^ (row & 7)) << 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(t_cv + off, b0, b1, b2, b3);
            mma_bf16_16816(ob[2 * np], pfb[0], pfb[1], pfb[2], pfb[3], b0, b1);
            mma_bf16_16816(ob[2 * np + 1], pfb[0], pfb[1], pfb[2], pfb[3], b2, b3);
            ldmatrix_x4_trans(t_sv + off, b0, b1, b2, b3);
            mma_bf16_16816(orr[2 * np], pfr[0], pfr[1], pfr[2], pfr[3], b0, b1);
            mma_bf16_16816(orr[2 * np + 1], pfr[0], pfr[1], pfr[2], pfr[3], b2, b3);
        }
        __syncwarp();
        issue(it + kTmNST - 1);
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    __syncthreads();  // all rings and tiles are drained: the work area becomes the merge area
    float* wacc = reinterpret_cast<float*>(tsm8);          // [W][16][LD]: base | residual accumulators
    float* wm = wacc + kTmWarps * 16 * kTmLD;              // [W][16]
    float* wl = wm + kTmWarps * 16;                        // [W][16], then 16 floats for the merged maxima
    float* fin = wl + kTmWarps * 16 + 96;                  // [16][2 D] merged head states
    const bool row0_used = gq < G, row1_used = gq + 8 < G;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int d = nt * 8 + tq * 2;
        if (row0_used) {
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq) * kTmLD + d]) = make_float2(ob[nt][0], ob[nt][1]);
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq) * kTmLD + D + d]) = make_float2(orr[nt][0], orr[nt][1]);
        }
        if (row1_used) {
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq + 8) * kTmLD + d]) = make_float2(ob[nt][2], ob[nt][3]);
            *reinterpret_cast<float2*>(&wacc[(warp * 16 + gq + 8) * kTmLD + D + d]) = make_float2(orr[nt][2], orr[nt][3]);
        }
    }
    if (tq == 0) {
        wm[warp * 16 + gq] = m0;
        wm[warp * 16 + gq + 8] = m1;
        wl[warp * 16 + gq] = l0;
        wl[warp * 16 + gq + 8] = l1;
    }
    __syncthreads();
    // weights of the eight warps per head, once; then the weighted sums of both accumulators
    float* hm = wl + kTmWarps * 16;  // [16] merged maximum, [16] merged l behind it
    if (tid < G) {
        float ms = -INFINITY, ls = 0.0f;
        for (int w = 0; w < kTmWarps; ++w) ms = fmaxf(ms, wm[w * 16 + tid]);
        for (int w = 0; w < kTmWarps; ++w) {
            const float mw = wm[w * 16 + tid];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - ms);
            ls += f * wl[w * 16 + tid];
            wm[w * 16 + tid] = f;
        }
        hm[tid] = ms;
        hm[16 + tid] = ls;
    }
    __syncthreads();
    for (int idx = tid; idx < G * 2 * D; idx += blockDim.x) {
        const int g = idx / (2 * D), c = idx - g * 2 * D;
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kTmWarps; ++w) o = fmaf(wm[w * 16 + g], wacc[(w * 16 + g) * kTmLD + c], o);
        fin[g * 2 * D + c] = o;
    }
    __syncthreads();
    // final transforms (:1323-1334): res <- T(res; res_post, res_pre); base += res; out = T(base; rot_post, rot_pre)
    for (int g = warp; g < G; g += kTmWarps) {
        float* fb = fin + g * 2 * D;
        turbo_transform_warp(fb + D, D, res_post, res_pre, lane);
        for (int i = lane; i < D; i += 32) fb[i] = fb[i] + fb[D + i];
        __syncwarp();
        turbo_transform_warp(fb, D, rot_post, rot_pre, lane);
    }
    __syncthreads();
    // one un-normalised state per head goes to the output, the cross-rank partial or the split scratch; the
    // weights handed to cta_merge_store are those of a single contributor (maximum and l as merged above)
    float* sm_ = hm + 32;  // [16] maxima, [16] l, [16] scratch of cta_merge_store
    if (tid < 16) {
        sm_[tid] = tid < G ? hm[tid] : -INFINITY;
        sm_[16 + tid] = tid < G ? hm[16 + tid] : 0.0f;
    }
    __syncthreads();
    cta_merge_store(a, fin, sm_, sm_ + 16, 1, 16, 0, G, item, kvh, split, 2 * D);
    __syncthreads();
    split_merge_store(a, item, kvh, &s_last, reinterpret_cast<float*>(tsm8));
}

inline int launch_turbo_mma(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const cudaError_t se = setup.ensure(attn_turbo_mma_kernel, device, smem_optin);
    if (se != cudaSuccess) return (int)se;
    attn_turbo_mma_kernel<<<grid, kTmWarps * 32, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace ggr
