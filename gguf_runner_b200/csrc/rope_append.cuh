// RoPE of q and k plus the KV-cache append for one item (one token) per CTA.
//
// Restates, for the device, apply_rope_qk (src/engine/runtime/inference.rs:1817-1874),
// rebuild_rope_cache (:1485-1523) and kv_write_token (:1877-1918). The
// rotation uses separately rounded multiplies and adds (no FMA contraction)
// so a rotated value differs from the reference's only through cos/sin.
#pragma once

#include "common.cuh"

namespace ggr {

enum RopeFlags : int {
    RF_ROTATE = 1,       // apply RoPE to q and k (else they are taken as already rotated)
    RF_WRITE_Q = 2,      // write rotated q to q_out (f32) and / or q_out_h (bf16)
    RF_APPEND = 4,       // store k, v into the cache row
    RF_WRITE_K = 8,      // write rotated k to k_out (apply_rope_qk called on its own)
};

struct RopeAppendArgs {
    RopeParams rope;
    KvView kv;
    Items items;
    int layer;
    int flags;
    int in_bf16;  // q/k/v inputs are bf16 instead of f32
    const void* q;
    const void* k;
    const void* v;
    float* q_out;             // [items][q_dim]
    __nv_bfloat16* q_out_h;   // optional bf16 copy, same shape
    float* k_out;             // [items][kv_dim]
    int shard_count;          // positions held locally (append only when pos is inside)
};

__device__ __forceinline__ float load_in(const void* p, int64_t idx, int in_bf16) {
    if (in_bf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
    return reinterpret_cast<const float*>(p)[idx];
}

// One rotated element of a head (NeoX split-half or adjacent pairs).
__device__ __forceinline__ float rope_elem(const void* x, int64_t base, int i, int D, const RopeParams& rp,
                                           const float* cs, const float* sn, int in_bf16) {
    if (rp.style == 0) {
        const int half = rp.rope_half;
        if (i < half) {
            float v0 = load_in(x, base + i, in_bf16), v1 = load_in(x, base + i + half, in_bf16);
            return __fsub_rn(__fmul_rn(v0, cs[i]), __fmul_rn(v1, sn[i]));
        } else if (i < rp.rope_dim) {
            int j = i - half;
            float v0 = load_in(x, base + j, in_bf16), v1 = load_in(x, base + i, in_bf16);
            return __fadd_rn(__fmul_rn(v0, sn[j]), __fmul_rn(v1, cs[j]));
        }
        return load_in(x, base + i, in_bf16);
    } else {
        int j = i >> 1;
        if ((i & 1) == 0) {
            float v0 = load_in(x, base + i, in_bf16), v1 = load_in(x, base + i + 1, in_bf16);
            return __fsub_rn(__fmul_rn(v0, cs[j]), __fmul_rn(v1, sn[j]));
        }
        float v0 = load_in(x, base + i - 1, in_bf16), v1 = load_in(x, base + i, in_bf16);
        return __fadd_rn(__fmul_rn(v0, sn[j]), __fmul_rn(v1, cs[j]));
    }
}

__device__ __forceinline__ int8_t q8_code(float x, float inv) {
    // src/engine/runtime/inference.rs:264-266: round half away from zero, clamp to +-127
    float r = roundf(__fmul_rn(x, inv));
    r = fminf(127.0f, fmaxf(-127.0f, r));
    return (int8_t)r;
}

// The attention kernel of a prefill call is launched with programmatic stream serialisation behind these kernels:
// signalling at the start lets its CTAs set themselves up while this grid drains (they wait for this grid's
// completion before reading anything). Without such a dependent the instruction does nothing.
__device__ __forceinline__ void rope_allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__global__ void __launch_bounds__(256) rope_append_kernel(RopeAppendArgs a) {
    extern __shared__ float sm[];
    rope_allow_dependents();
    const int D = a.kv.D, kv_dim = a.kv.kv_dim, q_dim = a.kv.Hq * D;
    const int half = a.rope.rope_half;
    float* cs = sm;
    float* sn = cs + half;
    float* krow = sn + half;
    float* vrow = krow + kv_dim;
    float* red = vrow + kv_dim;  // 2 * 8 partial maxima

    const int item = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    int seq, pos;
    a.items.get(item, seq, pos);

    if (a.flags & RF_ROTATE) {
        for (int i = tid; i < half; i += nt) {
            int axis = rope_axis(a.rope.layout, i, a.rope.sections);
            int coord = pos;
            if (a.rope.has_plan) {
                coord = pos < a.rope.plan_len ? a.rope.plan[pos * 3 + axis]
                                              : a.rope.next_text + (pos - a.rope.plan_len);
            }
            float val = __fmul_rn(__fmul_rn((float)coord, a.rope.freqs[i]), a.rope.fscale);
            float s, c;
            sincosf(val, &s, &c);
            cs[i] = c;
            sn[i] = s;
        }
        __syncthreads();
    }

    const int64_t qb = (int64_t)item * q_dim, kb = (int64_t)item * kv_dim;
    if (a.flags & RF_WRITE_Q) {
        for (int idx = tid; idx < q_dim; idx += nt) {
            int h = idx / D, i = idx - h * D;
            float r = (a.flags & RF_ROTATE) ? rope_elem(a.q, qb + (int64_t)h * D, i, D, a.rope, cs, sn, a.in_bf16)
                                            : load_in(a.q, qb + idx, a.in_bf16);
            if (a.rope.do_prescale) r = __fmul_rn(r, a.rope.q_prescale);
            if (a.q_out) a.q_out[qb + idx] = r;
            if (a.q_out_h) a.q_out_h[qb + idx] = __float2bfloat16_rn(r);
        }
    }
    if (!(a.flags & (RF_APPEND | RF_WRITE_K))) return;

    for (int idx = tid; idx < kv_dim; idx += nt) {
        int h = idx / D, i = idx - h * D;
        krow[idx] = (a.flags & RF_ROTATE) ? rope_elem(a.k, kb + (int64_t)h * D, i, D, a.rope, cs, sn, a.in_bf16)
                                          : load_in(a.k, kb + idx, a.in_bf16);
        if (a.flags & RF_APPEND) vrow[idx] = load_in(a.v, kb + idx, a.in_bf16);
    }
    __syncthreads();
    if (a.flags & RF_WRITE_K) {
        for (int idx = tid; idx < kv_dim; idx += nt) a.k_out[kb + idx] = krow[idx];
    }
    if (!(a.flags & RF_APPEND)) return;
    if (pos < a.kv.pos_begin || pos >= a.kv.pos_begin + a.shard_count) return;  // another rank owns this row

    const int64_t r = a.kv.row(seq, a.layer, pos);
    const int64_t off = r * kv_dim;
    switch (a.kv.fmt) {
        case KV_F32: {
            float* kc = reinterpret_cast<float*>(a.kv.k) + off;
            float* vc = reinterpret_cast<float*>(a.kv.v) + off;
            for (int idx = tid; idx < kv_dim; idx += nt) {
                kc[idx] = krow[idx];
                vc[idx] = vrow[idx];
            }
            break;
        }
        case KV_BF16: {
            __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(a.kv.k) + off;
            __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(a.kv.v) + off;
            for (int idx = tid; idx < kv_dim; idx += nt) {
                kc[idx] = __float2bfloat16_rn(krow[idx]);
                vc[idx] = __float2bfloat16_rn(vrow[idx]);
            }
            break;
        }
        case KV_Q8_ROW: {
            // one scale per row over all KV heads (src/engine/runtime/inference.rs:1906-1916)
            float mk = 0.0f, mv = 0.0f;
            for (int idx = tid; idx < kv_dim; idx += nt) {
                mk = fmaxf(mk, fabsf(krow[idx]));
                mv = fmaxf(mv, fabsf(vrow[idx]));
            }
            mk = warp_max(mk);
            mv = warp_max(mv);
            if ((tid & 31) == 0) {
                red[tid >> 5] = mk;
                red[8 + (tid >> 5)] = mv;
            }
            __syncthreads();
            mk = 0.0f;
            mv = 0.0f;
            for (int w = 0; w < (nt >> 5); ++w) {
                mk = fmaxf(mk, red[w]);
                mv = fmaxf(mv, red[8 + w]);
            }
            int8_t* kc = reinterpret_cast<int8_t*>(a.kv.k) + off;
            int8_t* vc = reinterpret_cast<int8_t*>(a.kv.v) + off;
            float invk = mk == 0.0f ? 0.0f : __fdiv_rn(127.0f, mk);
            float invv = mv == 0.0f ? 0.0f : __fdiv_rn(127.0f, mv);
            for (int idx = tid; idx < kv_dim; idx += nt) {
                kc[idx] = mk == 0.0f ? (int8_t)0 : q8_code(krow[idx], invk);
                vc[idx] = mv == 0.0f ? (int8_t)0 : q8_code(vrow[idx], invv);
            }
            if (tid == 0) {
                a.kv.ks[r] = mk == 0.0f ? 1.0f : __fdiv_rn(mk, 127.0f);
                a.kv.vs[r] = mv == 0.0f ? 1.0f : __fdiv_rn(mv, 127.0f);
            }
            break;
        }
        case KV_Q8_BLOCK32: {
            // one scale per 32 elements (src/engine/runtime/inference.rs:1888-1905)
            const int nb = kv_dim / 32;
            int8_t* kc = reinterpret_cast<int8_t*>(a.kv.k) + off;
            int8_t* vc = reinterpret_cast<int8_t*>(a.kv.v) + off;
            const int lane = tid & 31, warp = tid >> 5, nw = nt >> 5;
            for (int b = warp; b < nb; b += nw) {
                float xk = krow[b * 32 + lane], xv = vrow[b * 32 + lane];
                float mk = warp_max(fabsf(xk)), mv = warp_max(fabsf(xv));
                float invk = mk == 0.0f ? 0.0f : __fdiv_rn(127.0f, mk);
                float invv = mv == 0.0f ? 0.0f : __fdiv_rn(127.0f, mv);
                kc[b * 32 + lane] = mk == 0.0f ? (int8_t)0 : q8_code(xk, invk);
                vc[b * 32 + lane] = mv == 0.0f ? (int8_t)0 : q8_code(xv, invv);
                if (lane == 0) {
                    a.kv.ks[r * nb + b] = mk == 0.0f ? 1.0f : __fdiv_rn(mk, 127.0f);
                    a.kv.vs[r * nb + b] = mv == 0.0f ? 1.0f : __fdiv_rn(mv, 127.0f);
                }
            }
            break;
        }
    }
}

// ---- vectorised variant for the tensor-core prefill: bf16 inputs, bf16 cache, bf16 rotated q ----
// Same arithmetic as rope_append_kernel, but every thread moves 16-byte vectors (8 bf16) and a
// token needs one pass of the CTA: q, k and v tasks are spread over the 256 threads.

__device__ __forceinline__ void unpack8(const uint4& u, float f[8]) {
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
    f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
    f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}
__device__ __forceinline__ uint4 pack8(const float f[8]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c);
    u.w = *reinterpret_cast<uint32_t*>(&d);
    return u;
}

// Rotates head vector `vi` (8 elements) of a head starting at src; writes the result(s) to dst.
// NeoX: the thread owning a low-half vector also produces its partner in the high half.
__device__ __forceinline__ void rope_vec8(const __nv_bfloat16* src, __nv_bfloat16* dst, int vi, const RopeParams& rp,
                                          const float* cs, const float* sn, float scale, bool do_scale) {
    const int e0 = vi * 8;
    const uint4 u = *reinterpret_cast<const uint4*>(src + e0);
    float x[8];
    unpack8(u, x);
    if (rp.style == 0) {
        const int half = rp.rope_half;
        if (e0 < half) {
            const uint4 w = *reinterpret_cast<const uint4*>(src + e0 + half);
            float y[8], lo[8], hi[8];
            unpack8(w, y);
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                const float c = cs[e0 + p], s = sn[e0 + p];
                lo[p] = __fsub_rn(__fmul_rn(x[p], c), __fmul_rn(y[p], s));
                hi[p] = __fadd_rn(__fmul_rn(x[p], s), __fmul_rn(y[p], c));
                if (do_scale) {
                    lo[p] = __fmul_rn(lo[p], scale);
                    hi[p] = __fmul_rn(hi[p], scale);
                }
            }
            *reinterpret_cast<uint4*>(dst + e0) = pack8(lo);
            *reinterpret_cast<uint4*>(dst + e0 + half) = pack8(hi);
        } else if (e0 >= rp.rope_dim) {
            if (do_scale) {
#pragma unroll
                for (int p = 0; p < 8; ++p) x[p] = __fmul_rn(x[p], scale);
                *reinterpret_cast<uint4*>(dst + e0) = pack8(x);
            } else {
                *reinterpret_cast<uint4*>(dst + e0) = u;
            }
        }
    } else {
        float r[8];
#pragma unroll
        for (int p = 0; p < 8; p += 2) {
            const int j = (e0 + p) >> 1;
            const float c = cs[j], s = sn[j];
            r[p] = __fsub_rn(__fmul_rn(x[p], c), __fmul_rn(x[p + 1], s));
            r[p + 1] = __fadd_rn(__fmul_rn(x[p], s), __fmul_rn(x[p + 1], c));
            if (do_scale) {
                r[p] = __fmul_rn(r[p], scale);
                r[p + 1] = __fmul_rn(r[p + 1], scale);
            }
        }
        *reinterpret_cast<uint4*>(dst + e0) = pack8(r);
    }
}

inline bool rope_append_fast_ok(const RopeAppendArgs& a) {
    const int D = a.kv.D;
    return a.in_bf16 && a.kv.fmt == KV_BF16 && a.q_out_h && !a.q_out && !a.k_out &&
           a.flags == (RF_ROTATE | RF_WRITE_Q | RF_APPEND) && D % 8 == 0 && a.rope.rope_half <= 128 &&
           ((a.rope.style == 1 && a.rope.rope_dim == D) || (a.rope.style == 0 && a.rope.rope_half % 8 == 0 && a.rope.rope_dim % 8 == 0)) &&
           a.kv.pos_begin == 0;
}

__global__ void __launch_bounds__(256) rope_append_bf16_kernel(RopeAppendArgs a) {
    __shared__ float cs[128], sn[128];
    rope_allow_dependents();
    const int D = a.kv.D, kv_dim = a.kv.kv_dim, Hq = a.kv.Hq, Hkv = a.kv.Hkv, q_dim = Hq * D;
    const int half = a.rope.rope_half;
    const int item = blockIdx.x, tid = threadIdx.x;
    int seq, pos;
    a.items.get(item, seq, pos);
    if (tid < half) {
        const int axis = rope_axis(a.rope.layout, tid, a.rope.sections);
        int coord = pos;
        if (a.rope.has_plan)
            coord = pos < a.rope.plan_len ? a.rope.plan[pos * 3 + axis] : a.rope.next_text + (pos - a.rope.plan_len);
        const float val = __fmul_rn(__fmul_rn((float)coord, a.rope.freqs[tid]), a.rope.fscale);
        float s, c;
        sincosf(val, &s, &c);
        cs[tid] = c;
        sn[tid] = s;
    }
    __syncthreads();
    const int vph = D / 8;  // vectors per head
    const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(a.q) + (int64_t)item * q_dim;
    const __nv_bfloat16* k = reinterpret_cast<const __nv_bfloat16*>(a.k) + (int64_t)item * kv_dim;
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(a.v) + (int64_t)item * kv_dim;
    __nv_bfloat16* qo = a.q_out_h + (int64_t)item * q_dim;
    const int64_t off = a.kv.row(seq, a.layer, pos) * kv_dim;
    __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(a.kv.k) + off;
    __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(a.kv.v) + off;
    const int nq = Hq * vph, nk = Hkv * vph, total = nq + 2 * nk;
    for (int task = tid; task < total; task += blockDim.x) {
        if (task < nq) {
            const int h = task / vph, vi = task - h * vph;
            rope_vec8(q + h * D, qo + h * D, vi, a.rope, cs, sn, a.rope.q_prescale, a.rope.do_prescale != 0);
        } else if (task < nq + nk) {
            const int t2 = task - nq, h = t2 / vph, vi = t2 - h * vph;
            rope_vec8(k + h * D, kc + h * D, vi, a.rope, cs, sn, 1.0f, false);
        } else {
            const int t2 = task - nq - nk;
            *reinterpret_cast<uint4*>(vc + t2 * 8) = *reinterpret_cast<const uint4*>(v + t2 * 8);
        }
    }
}

// ---- vectorised general variant -------------------------------------------------------------------
// Same results as rope_append_kernel for f32 or bf16 inputs and every cache format, with 8-element
// (16 / 32 byte) loads and stores and one task per thread instead of element loops whose loads the
// compiler has to serialise. Needs the rotated span to be a multiple of 8 elements.

template <typename TIn>
__device__ __forceinline__ void load8_in(const TIn* p, float x[8]);
template <>
__device__ __forceinline__ void load8_in<float>(const float* p, float x[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_in<__nv_bfloat16>(const __nv_bfloat16* p, float x[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), x);
}
__device__ __forceinline__ void store8_f32(float* p, const float x[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

// Rotates vector vi of a head. Returns the number of result vectors (0, 1 or 2): r0 belongs at
// element e0, r1 (NeoX partner) at e0 + rope_half.
template <typename TIn>
__device__ __forceinline__ int rope_task8(const TIn* head, int vi, const RopeParams& rp, const float* cs, const float* sn,
                                          bool rotate, float r0[8], float r1[8]) {
    const int e0 = vi * 8;
    float x[8];
    if (!rotate) {
        load8_in<TIn>(head + e0, r0);
        return 1;
    }
    if (rp.style == 0) {
        const int half = rp.rope_half;
        if (e0 < half) {
            float y[8];
            load8_in<TIn>(head + e0, x);
            load8_in<TIn>(head + e0 + half, y);
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                const float c = cs[e0 + p], s = sn[e0 + p];
                r0[p] = __fsub_rn(__fmul_rn(x[p], c), __fmul_rn(y[p], s));
                r1[p] = __fadd_rn(__fmul_rn(x[p], s), __fmul_rn(y[p], c));
            }
            return 2;
        }
        if (e0 < rp.rope_dim) return 0;  // produced by the low-half partner
        load8_in<TIn>(head + e0, r0);
        return 1;
    }
    load8_in<TIn>(head + e0, x);
#pragma unroll
    for (int p = 0; p < 8; p += 2) {
        const int j = (e0 + p) >> 1;
        const float c = cs[j], s = sn[j];
        r0[p] = __fsub_rn(__fmul_rn(x[p], c), __fmul_rn(x[p + 1], s));
        r0[p + 1] = __fadd_rn(__fmul_rn(x[p], s), __fmul_rn(x[p + 1], c));
    }
    return 1;
}

inline bool rope_append_vec_ok(const RopeAppendArgs& a) {
    // adjacent pairs: the vector kernels rotate every pair of the head, so the rotated span must be the whole head
    const bool span_ok = (a.rope.style == 1 && a.rope.rope_dim == a.kv.D) ||
                         (a.rope.style == 0 && a.rope.rope_half % 8 == 0 && a.rope.rope_dim % 8 == 0);
    return span_ok && a.kv.D % 8 == 0 && a.kv.fmt != KV_Q8_BLOCK32;
}

template <typename TIn>
__global__ void __launch_bounds__(256) rope_append_vec_kernel(RopeAppendArgs a) {
    rope_allow_dependents();
    extern __shared__ float sm[];
    const int D = a.kv.D, kv_dim = a.kv.kv_dim, Hq = a.kv.Hq, Hkv = a.kv.Hkv, q_dim = Hq * D;
    const int half = a.rope.rope_half;
    float* cs = sm;
    float* sn = cs + half;
    float* krow = sm + ((2 * half + 3) & ~3);  // 16-byte aligned rows
    float* vrow = krow + kv_dim;
    float* red = vrow + kv_dim;
    const int item = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    int seq, pos;
    a.items.get(item, seq, pos);
    const bool rotate = (a.flags & RF_ROTATE) != 0;
    if (rotate) {
        for (int i = tid; i < half; i += nt) {
            const int axis = rope_axis(a.rope.layout, i, a.rope.sections);
            int coord = pos;
            if (a.rope.has_plan)
                coord = pos < a.rope.plan_len ? a.rope.plan[pos * 3 + axis] : a.rope.next_text + (pos - a.rope.plan_len);
            const float val = __fmul_rn(__fmul_rn((float)coord, a.rope.freqs[i]), a.rope.fscale);
            float s, c;
            sincosf(val, &s, &c);
            cs[i] = c;
            sn[i] = s;
        }
        __syncthreads();
    }
    const int vph = D / 8;
    const TIn* q = reinterpret_cast<const TIn*>(a.q) + (int64_t)item * q_dim;
    const TIn* k = reinterpret_cast<const TIn*>(a.k) + (int64_t)item * kv_dim;
    const TIn* v = reinterpret_cast<const TIn*>(a.v) + (int64_t)item * kv_dim;
    const bool do_q = (a.flags & RF_WRITE_Q) != 0;
    const bool do_k = (a.flags & (RF_APPEND | RF_WRITE_K)) != 0;
    const bool do_v = (a.flags & RF_APPEND) != 0;
    const int nq = do_q ? Hq * vph : 0, nk = do_k ? Hkv * vph : 0, nv = do_v ? Hkv * vph : 0;
    for (int task = tid; task < nq + nk + nv; task += nt) {
        float r0[8], r1[8];
        if (task < nq) {
            const int h = task / vph, vi = task - h * vph;
            const int n = rope_task8<TIn>(q + h * D, vi, a.rope, cs, sn, rotate, r0, r1);
            const int64_t o = (int64_t)item * q_dim + h * D + vi * 8;
            for (int r = 0; r < n; ++r) {
                float* x = r == 0 ? r0 : r1;
                const int64_t oo = o + (r == 0 ? 0 : half);
                if (a.rope.do_prescale) {
#pragma unroll
                    for (int p = 0; p < 8; ++p) x[p] = __fmul_rn(x[p], a.rope.q_prescale);
                }
                if (a.q_out) store8_f32(a.q_out + oo, x);
                if (a.q_out_h) *reinterpret_cast<uint4*>(a.q_out_h + oo) = pack8(x);
            }
        } else if (task < nq + nk) {
            const int t2 = task - nq, h = t2 / vph, vi = t2 - h * vph;
            const int n = rope_task8<TIn>(k + h * D, vi, a.rope, cs, sn, rotate, r0, r1);
            if (n >= 1) store8_f32(krow + h * D + vi * 8, r0);
            if (n == 2) store8_f32(krow + h * D + vi * 8 + half, r1);
        } else {
            const int t2 = task - nq - nk;
            load8_in<TIn>(v + t2 * 8, r0);
            store8_f32(vrow + t2 * 8, r0);
        }
    }
    if (!do_k) return;
    __syncthreads();
    const int nvec = kv_dim / 8;
    if (a.flags & RF_WRITE_K) {
        float* ko = a.k_out + (int64_t)item * kv_dim;
        for (int t2 = tid; t2 < nvec; t2 += nt) store8_f32(ko + t2 * 8, krow + t2 * 8);
    }
    if (!do_v) return;
    if (pos < a.kv.pos_begin || pos >= a.kv.pos_begin + a.shard_count) return;  // another rank owns this row
    const int64_t r = a.kv.row(seq, a.layer, pos);
    const int64_t off = r * kv_dim;
    if (a.kv.fmt == KV_F32) {
        float* kc = reinterpret_cast<float*>(a.kv.k) + off;
        float* vc = reinterpret_cast<float*>(a.kv.v) + off;
        for (int t2 = tid; t2 < nvec; t2 += nt) {
            store8_f32(kc + t2 * 8, krow + t2 * 8);
            store8_f32(vc + t2 * 8, vrow + t2 * 8);
        }
    } else if (a.kv.fmt == KV_BF16) {
        __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(a.kv.k) + off;
        __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(a.kv.v) + off;
        for (int t2 = tid; t2 < nvec; t2 += nt) {
            *reinterpret_cast<uint4*>(kc + t2 * 8) = pack8(krow + t2 * 8);
            *reinterpret_cast<uint4*>(vc + t2 * 8) = pack8(vrow + t2 * 8);
        }
    } else {  // KV_Q8_ROW: one scale per row over all KV heads (src/engine/runtime/inference.rs:1906-1916)
        float mk = 0.0f, mv = 0.0f;
        for (int idx = tid; idx < kv_dim; idx += nt) {
            mk = fmaxf(mk, fabsf(krow[idx]));
            mv = fmaxf(mv, fabsf(vrow[idx]));
        }
        mk = warp_max(mk);
        mv = warp_max(mv);
        if ((tid & 31) == 0) {
            red[tid >> 5] = mk;
            red[8 + (tid >> 5)] = mv;
        }
        __syncthreads();
        mk = 0.0f;
        mv = 0.0f;
        for (int w = 0; w < (nt >> 5); ++w) {
            mk = fmaxf(mk, red[w]);
            mv = fmaxf(mv, red[8 + w]);
        }
        const float invk = mk == 0.0f ? 0.0f : __fdiv_rn(127.0f, mk);
        const float invv = mv == 0.0f ? 0.0f : __fdiv_rn(127.0f, mv);
        int8_t* kc = reinterpret_cast<int8_t*>(a.kv.k) + off;
        int8_t* vc = reinterpret_cast<int8_t*>(a.kv.v) + off;
        for (int t2 = tid; t2 < nvec; t2 += nt) {
            uint32_t kw[2] = {0, 0}, vw[2] = {0, 0};
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                const int8_t kq = mk == 0.0f ? (int8_t)0 : q8_code(krow[t2 * 8 + p], invk);
                const int8_t vq = mv == 0.0f ? (int8_t)0 : q8_code(vrow[t2 * 8 + p], invv);
                kw[p >> 2] |= (uint32_t)(uint8_t)kq << (8 * (p & 3));
                vw[p >> 2] |= (uint32_t)(uint8_t)vq << (8 * (p & 3));
            }
            *reinterpret_cast<uint2*>(kc + t2 * 8) = make_uint2(kw[0], kw[1]);
            *reinterpret_cast<uint2*>(vc + t2 * 8) = make_uint2(vw[0], vw[1]);
        }
        if (tid == 0) {
            a.kv.ks[r] = mk == 0.0f ? 1.0f : __fdiv_rn(mk, 127.0f);
            a.kv.vs[r] = mv == 0.0f ? 1.0f : __fdiv_rn(mv, 127.0f);
        }
    }
}

// ---- pre-attention fixups: Qwen2 biases and per-head RMS QK-norm --------------------------------------
// Device counterpart of qkv_bias_and_norm (src/engine/runtime/inference.rs:2535-2572) and
// rmsnorm_per_head_gemma_inplace (src/engine/kernels/math.rs:164-184): q/k/v (+ bias), then
// x = weight * (x / sqrt(mean(x^2) + eps)) per head of q and k. One CTA per token, one warp per head;
// results go to f32 scratch rows that the rope/append (or fused decode) kernels then read.
struct FixupArgs {
    const void* q;
    const void* k;
    const void* v;
    int in_bf16;
    const float* q_bias;  // [q_dim] or null
    const float* k_bias;  // [kv_dim]
    const float* v_bias;  // [kv_dim]
    const float* q_norm;  // [D] or null
    const float* k_norm;  // [D]
    float eps;
    int Hq, Hkv, D;
    float* q_out;
    float* k_out;
    float* v_out;
};

__global__ void __launch_bounds__(256) qkv_fixup_kernel(FixupArgs a) {
    const int item = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int D = a.D, q_dim = a.Hq * D, kv_dim = a.Hkv * D;
    for (int hh = warp; hh < a.Hq + a.Hkv; hh += nw) {
        const bool is_q = hh < a.Hq;
        const int h = is_q ? hh : hh - a.Hq;
        const int64_t base = (int64_t)item * (is_q ? q_dim : kv_dim) + (int64_t)h * D;
        const void* src = is_q ? a.q : a.k;
        const float* bias = is_q ? a.q_bias : a.k_bias;
        const float* w = is_q ? a.q_norm : a.k_norm;
        float* dst = (is_q ? a.q_out : a.k_out) + base;
        float ss = 0.0f;
        for (int j = lane; j < D; j += 32) {
            float x = load_in(src, base + j, a.in_bf16);
            if (bias) x = __fadd_rn(x, bias[h * D + j]);
            dst[j] = x;
            ss = fmaf(x, x, ss);
        }
        if (w) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
            __syncwarp();
            for (int j = lane; j < D; j += 32) dst[j] = __fmul_rn(w[j], __fmul_rn(inv, dst[j]));
        }
    }
    for (int idx = threadIdx.x; idx < kv_dim; idx += blockDim.x) {
        float x = load_in(a.v, (int64_t)item * kv_dim + idx, a.in_bf16);
        if (a.v_bias) x = __fadd_rn(x, a.v_bias[idx]);
        a.v_out[(int64_t)item * kv_dim + idx] = x;
    }
}

}  // namespace ggr
