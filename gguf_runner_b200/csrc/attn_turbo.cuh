// TurboQuant KV cache on the device: 2-bit codes + 1 residual sign bit per element, sigma and residual norm per
// (row, kv head). Device counterpart of the Turbo arms of kv_write_token and attention_token
// (src/engine/runtime/inference.rs:885-982 write / query preparation, :1246-1334 score, value sum and final
// transforms; sign tables :370-395).
//
// Layout (identical to the reference, per sequence and layer): element e = row * kv_dim + kv_head * D + i;
// codes kv.k / kv.v: byte e / 4, bits 2 * (e & 3); sign bits kv.k_sign / kv.v_sign: byte e / 8, bit e & 7
// (1 = the projected residual is >= 0); kv.ks / kv.vs (sigma) and kv.k_rn / kv.v_rn (residual norm): index
// row * Hkv + kv_head. Transform sign tables kv.turbo_signs: [slot][layer][kv_head][D / 8], bit 1 = negate.
//
// The append is bit-exact against the CPU restatement: the butterflies are the same additions in the same
// stage order, the two norms are summed sequentially by one lane, and every product that the reference rounds
// separately is rounded separately here. The attention kernel computes in f32 on the CUDA cores: the score is
// sigma * sum(q_r * centroid) + rho * sum(+-q_p), so the 2-bit table lookup costs one multiply-add per element.
#pragma once

#include "attn_simt.cuh"
#include "common.cuh"
#include "rope_append.cuh"

namespace ggr {

__device__ __constant__ float kTurboCentroid[4] = {-1.510417f, -0.45278f, 0.45278f, 1.510417f};
constexpr float kTurboThreshold = 0.9815985f;

__device__ __forceinline__ const unsigned char* turbo_sign_slot(const KvView& kv, int slot, int layer, int kvh) {
    const int bytes = kv.D / 8;
    return kv.turbo_signs + ((size_t)slot * kv.n_layers * kv.Hkv + (size_t)layer * kv.Hkv + kvh) * bytes;
}

// sign_b . FWHT(sign_a . x) on n floats in shared memory, by one warp. The FWHT (scaled by 1 / sqrt(n)) is
// skipped when n is not a power of two, as in the reference (:822-825).
__device__ __forceinline__ void turbo_transform_warp(float* x, int n, const unsigned char* first,
                                                     const unsigned char* second, int lane) {
    for (int i = lane; i < n; i += 32)
        if ((first[i >> 3] >> (i & 7)) & 1) x[i] = -x[i];
    __syncwarp();
    if ((n & (n - 1)) == 0) {
        for (int width = 1; width < n; width <<= 1) {
            for (int p = lane; p < n / 2; p += 32) {
                const int i = p & (width - 1), base = (p - i) * 2;
                const float a = x[base + i], b = x[base + i + width];
                x[base + i] = __fadd_rn(a, b);
                x[base + i + width] = __fsub_rn(a, b);
            }
            __syncwarp();
        }
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)n));
        for (int i = lane; i < n; i += 32) x[i] = __fmul_rn(x[i], scale);
        __syncwarp();
    }
    for (int i = lane; i < n; i += 32)
        if ((second[i >> 3] >> (i & 7)) & 1) x[i] = -x[i];
    __syncwarp();
}

// sqrt(sum x^2), summed in index order by lane 0 (src/engine/kernels/math.rs:467-473) and broadcast
__device__ __forceinline__ float turbo_l2_norm_warp(const float* x, int n, int lane) {
    float r = 0.0f;
    if (lane == 0) {
        float ss = 0.0f;
        for (int i = 0; i < n; ++i) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
        r = __fsqrt_rn(ss);
    }
    return __shfl_sync(0xffffffffu, r, 0);
}

struct TurboAppendArgs {
    KvView kv;
    Items items;
    int layer;
    const float* k_rot;  // [items][kv_dim] rotated keys (f32)
    const void* v;       // [items][kv_dim] values, f32 or bf16
    int v_bf16;
    int shard_count;
};

// grid (items, Hkv), 64 threads: warp 0 quantises the K head, warp 1 the V head (:885-952)
__global__ void __launch_bounds__(64) turbo_append_kernel(TurboAppendArgs a) {
    extern __shared__ float tsm[];
    const int D = a.kv.D, kv_dim = a.kv.kv_dim;
    const int item = blockIdx.x, kvh = blockIdx.y, lane = threadIdx.x & 31, which = threadIdx.x >> 5;
    int seq, pos;
    a.items.get(item, seq, pos);
    if (pos < a.kv.pos_begin || pos >= a.kv.pos_begin + a.shard_count) return;  // another rank owns this row
    float* rot = tsm + which * 2 * D;
    float* res = rot + D;
    const int64_t in_off = (int64_t)item * kv_dim + (int64_t)kvh * D;
    for (int i = lane; i < D; i += 32) rot[i] = which == 0 ? a.k_rot[in_off + i] : load_in(a.v, in_off + i, a.v_bf16);
    __syncwarp();
    turbo_transform_warp(rot, D, turbo_sign_slot(a.kv, 0, a.layer, kvh), turbo_sign_slot(a.kv, 1, a.layer, kvh), lane);

    const int64_t row = a.kv.row(seq, a.layer, pos);
    const int64_t eo = row * kv_dim + (int64_t)kvh * D, aux = row * a.kv.Hkv + kvh;
    unsigned char* base = reinterpret_cast<unsigned char*>(which == 0 ? a.kv.k : a.kv.v) + eo / 4;
    unsigned char* sign = (which == 0 ? a.kv.k_sign : a.kv.v_sign) + eo / 8;
    float* scale_out = (which == 0 ? a.kv.ks : a.kv.vs) + aux;
    float* rnorm_out = (which == 0 ? a.kv.k_rn : a.kv.v_rn) + aux;

    const float sigma = __fdiv_rn(turbo_l2_norm_warp(rot, D, lane), __fsqrt_rn((float)D));
    if (lane == 0) *scale_out = sigma;
    if (sigma == 0.0f) {
        if (lane == 0) *rnorm_out = 0.0f;
        for (int b = lane; b < D / 4; b += 32) base[b] = 0;
        for (int b = lane; b < D / 8; b += 32) sign[b] = 0xff;
        return;
    }
    const float inv_sigma = __fdiv_rn(1.0f, sigma);
    for (int b = lane; b < D / 4; b += 32) {
        unsigned packed = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float value = rot[4 * b + k], x = __fmul_rn(value, inv_sigma);
            const int code = x < -kTurboThreshold ? 0 : (x < 0.0f ? 1 : (x < kTurboThreshold ? 2 : 3));
            res[4 * b + k] = __fsub_rn(value, __fmul_rn(kTurboCentroid[code], sigma));
            packed |= (unsigned)code << (2 * k);
        }
        base[b] = (unsigned char)packed;
    }
    __syncwarp();
    const float gamma = turbo_l2_norm_warp(res, D, lane);
    if (lane == 0) *rnorm_out = gamma;
    if (gamma == 0.0f) {
        for (int b = lane; b < D / 8; b += 32) sign[b] = 0xff;
        return;
    }
    for (int i = lane; i < D; i += 32) res[i] = __fdiv_rn(res[i], gamma);
    __syncwarp();
    turbo_transform_warp(res, D, turbo_sign_slot(a.kv, 2, a.layer, kvh), turbo_sign_slot(a.kv, 3, a.layer, kvh), lane);
    for (int b = lane; b < D / 8; b += 32) {
        unsigned bits = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) bits |= (res[8 * b + k] >= 0.0f ? 1u : 0u) << k;
        sign[b] = (unsigned char)bits;
    }
}

constexpr int kTurboWarps = 4;
constexpr int kTurboGroups = kTurboWarps * 4;  // eight lanes share a key

// shared memory of attn_turbo_kernel, in floats
inline size_t turbo_attn_smem_floats(int D, int G, int GH, int n_split) {
    const size_t prep = (size_t)2 * G * D;                                 // rotated and projected queries
    const size_t part = (size_t)kTurboGroups * GH * (2 * D + 2);           // per-group accumulators, m, l
    const size_t fin = (size_t)GH * 2 * D + 3 * GH + 8;                    // merged head states
    const size_t merge = n_split > 1 ? (size_t)2 * G * n_split + 2 * G + split_merge_sub_floats(G, D) : 0;  // split merge weights, sub-results
    return prep + (part + fin > merge ? part + fin : merge);
}

// Split-KV attention over a TurboQuant cache: grid (n_split, Hkv, items), four warps. Every group of eight
// lanes takes one key at a time; a lane owns D / 8 consecutive elements of it. GH query heads of the KV head
// are carried per pass over the keys.
template <int D, int GH>
__global__ void __launch_bounds__(kTurboWarps * 32) attn_turbo_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smf[];
    __shared__ int s_last;
    constexpr int EPL = D / 8;     // elements per lane
    constexpr int CB = EPL / 4;    // code bytes per lane
    constexpr int SB = EPL / 8;    // sign bytes per lane
    const int G = a.kv.G, Hkv = a.kv.Hkv, kv_dim = a.kv.kv_dim;
    const int split = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int grp = warp * 4 + (lane >> 3), sl = lane & 7;
    const unsigned gmask = 0xffu << (lane & 24);

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

    float* qr = smf;               // [G][D]
    float* qp = qr + G * D;        // [G][D]
    float* work = qp + G * D;
    float* pacc = work;                                          // [groups][GH][2][D]
    float* pm = pacc + kTurboGroups * GH * 2 * D;                // [groups][GH]
    float* pl = pm + kTurboGroups * GH;                          // [groups][GH]
    float* fin = pl + kTurboGroups * GH;                         // [GH][2][D]
    float* wm = fin + GH * 2 * D;                                // [GH], then wl [GH], wx [GH]
    float* wl = wm + GH;

    // query preparation (:954-968): q_r = T(q; rot_pre, rot_post), q_p = T(q_r; res_pre, res_post)
    const unsigned char* rot_pre = turbo_sign_slot(a.kv, 0, a.layer, kvh);
    const unsigned char* rot_post = turbo_sign_slot(a.kv, 1, a.layer, kvh);
    const unsigned char* res_pre = turbo_sign_slot(a.kv, 2, a.layer, kvh);
    const unsigned char* res_post = turbo_sign_slot(a.kv, 3, a.layer, kvh);
    const float* qsrc = a.q + ((int64_t)item * a.kv.Hq + (int64_t)kvh * G) * D;
    for (int g = warp; g < G; g += kTurboWarps) {
        for (int i = lane; i < D; i += 32) qr[g * D + i] = qsrc[(int64_t)g * D + i];
        __syncwarp();
        turbo_transform_warp(qr + g * D, D, rot_pre, rot_post, lane);
        for (int i = lane; i < D; i += 32) qp[g * D + i] = qr[g * D + i];
        __syncwarp();
        turbo_transform_warp(qp + g * D, D, res_pre, res_post, lane);
    }
    __syncthreads();

    const unsigned char* kbase = reinterpret_cast<const unsigned char*>(a.kv.k);
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(a.kv.v);
    const float rho_unit = __fsqrt_rn(__fdiv_rn(1.57079632679489661923f, (float)D));  // :975-982

    for (int g0 = 0; g0 < G; g0 += GH) {
        float qrr[GH][EPL], qpr[GH][EPL], bacc[GH][EPL], racc[GH][EPL], m[GH], l[GH];
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            m[h] = -INFINITY;
            l[h] = 0.0f;
            const bool hv = g0 + h < G;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                qrr[h][e] = hv ? qr[(g0 + h) * D + sl * EPL + e] : 0.0f;
                qpr[h][e] = hv ? qp[(g0 + h) * D + sl * EPL + e] : 0.0f;
                bacc[h][e] = 0.0f;
                racc[h][e] = 0.0f;
            }
        }
        for (int t = k0 + grp; t < k1; t += kTurboGroups) {
            const int64_t row = row0 + t;
            const int64_t eo = row * kv_dim + (int64_t)kvh * D + sl * EPL, aux = row * Hkv + kvh;
            unsigned char kc[CB], ksg[SB], vc[CB], vsg[SB];
#pragma unroll
            for (int b = 0; b < CB; ++b) {
                kc[b] = kbase[eo / 4 + b];
                vc[b] = vbase[eo / 4 + b];
            }
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                ksg[b] = a.kv.k_sign[eo / 8 + b];
                vsg[b] = a.kv.v_sign[eo / 8 + b];
            }
            const float k_sigma = a.kv.ks[aux], k_rho = a.kv.k_rn[aux] * rho_unit;
            const float v_sigma = a.kv.vs[aux], v_rho = a.kv.v_rn[aux] * rho_unit;
            // scores (:1246-1269)
            float sc[GH];
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                float cs = 0.0f, rs = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const int code = (kc[e >> 2] >> (2 * (e & 3))) & 3;
                    cs = fmaf(qrr[h][e], kTurboCentroid[code], cs);
                    rs += ((ksg[e >> 3] >> (e & 7)) & 1) ? qpr[h][e] : -qpr[h][e];
                }
                float sv = fmaf(k_sigma, cs, k_rho * rs);
                sv += __shfl_xor_sync(gmask, sv, 1);
                sv += __shfl_xor_sync(gmask, sv, 2);
                sv += __shfl_xor_sync(gmask, sv, 4);
                sc[h] = sv * a.score_scale;
            }
            // online softmax and value sums (:1284-1306)
            float cv[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) cv[e] = kTurboCentroid[(vc[e >> 2] >> (2 * (e & 3))) & 3] * v_sigma;
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                if (sc[h] > m[h]) {
                    const float al = exp2f(m[h] - sc[h]);  // 0 on the first key
                    l[h] *= al;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) {
                        bacc[h][e] *= al;
                        racc[h][e] *= al;
                    }
                    m[h] = sc[h];
                }
                const float p = exp2f(sc[h] - m[h]);
                l[h] += p;
                const float pr = p * v_rho;
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    bacc[h][e] = fmaf(p, cv[e], bacc[h][e]);
                    racc[h][e] += ((vsg[e >> 3] >> (e & 7)) & 1) ? pr : -pr;
                }
            }
        }
        // the sixteen key groups of the CTA merge through shared memory
#pragma unroll
        for (int h = 0; h < GH; ++h) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                pacc[((grp * GH + h) * 2 + 0) * D + sl * EPL + e] = bacc[h][e];
                pacc[((grp * GH + h) * 2 + 1) * D + sl * EPL + e] = racc[h][e];
            }
            if (sl == 0) {
                pm[grp * GH + h] = m[h];
                pl[grp * GH + h] = l[h];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < GH * 2 * D; idx += blockDim.x) {
            const int h = idx / (2 * D), rem = idx - h * 2 * D;
            float ms = -INFINITY;
            for (int gi = 0; gi < kTurboGroups; ++gi) ms = fmaxf(ms, pm[gi * GH + h]);
            float o = 0.0f;
            for (int gi = 0; gi < kTurboGroups; ++gi) {
                const float mg = pm[gi * GH + h];
                const float f = mg == -INFINITY ? 0.0f : exp2f(mg - ms);
                o = fmaf(f, pacc[(gi * GH + h) * 2 * D + rem], o);
            }
            fin[h * 2 * D + rem] = o;
        }
        if (tid < GH) {
            float ms = -INFINITY, ls = 0.0f;
            for (int gi = 0; gi < kTurboGroups; ++gi) ms = fmaxf(ms, pm[gi * GH + tid]);
            for (int gi = 0; gi < kTurboGroups; ++gi) {
                const float mg = pm[gi * GH + tid];
                ls += mg == -INFINITY ? 0.0f : exp2f(mg - ms) * pl[gi * GH + tid];
            }
            wm[tid] = ms;
            wl[tid] = ls;
        }
        __syncthreads();
        // final transforms (:1323-1334): res <- T(res; res_post, res_pre); base += res; out = T(base; rot_post, rot_pre)
        if (warp < GH) {
            float* fb = fin + warp * 2 * D;
            turbo_transform_warp(fb + D, D, res_post, res_pre, lane);
            for (int i = lane; i < D; i += 32) fb[i] = fb[i] + fb[D + i];
            __syncwarp();
            turbo_transform_warp(fb, D, rot_post, rot_pre, lane);
        }
        __syncthreads();
        // one un-normalised state per head goes to the output, the cross-rank partial or the split scratch
        cta_merge_store(a, fin, wm, wl, 1, GH, g0, min(GH, G - g0), item, kvh, split, 2 * D);
        __syncthreads();
    }
    split_merge_store(a, item, kvh, &s_last, work);
}

template <int D, int GH>
inline int launch_turbo_inst(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const cudaError_t se = setup.ensure(attn_turbo_kernel<D, GH>, device, smem_optin);
    if (se != cudaSuccess) return (int)se;
    attn_turbo_kernel<D, GH><<<grid, kTurboWarps * 32, smem, stream>>>(a);
    return (int)cudaGetLastError();
}

// two heads per pass when the accumulators fit in registers (head_dim 256 carries one)
inline int turbo_heads_per_pass(int G, int D) { return (G % 2 == 0 && D <= 128) ? 2 : 1; }

inline int launch_turbo_attention(const AttnArgs& a, dim3 grid, size_t smem, int smem_optin, int device,
                                  cudaStream_t stream) {
    const int gh = turbo_heads_per_pass(a.kv.G, a.kv.D);
    switch (a.kv.D) {
        case 64: return gh == 2 ? launch_turbo_inst<64, 2>(a, grid, smem, smem_optin, device, stream)
                                : launch_turbo_inst<64, 1>(a, grid, smem, smem_optin, device, stream);
        case 128: return gh == 2 ? launch_turbo_inst<128, 2>(a, grid, smem, smem_optin, device, stream)
                                 : launch_turbo_inst<128, 1>(a, grid, smem, smem_optin, device, stream);
        case 256: return launch_turbo_inst<256, 1>(a, grid, smem, smem_optin, device, stream);
        default: return (int)cudaErrorNotSupported;
    }
}

}  // namespace ggr
