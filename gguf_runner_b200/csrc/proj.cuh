// The matmuls either side of the attention path: q / k / v projections in front of it and the output
// projection behind it (src/engine/runtime/inference.rs:3144-3476 and :3520-3527; one activation row against
// every weight row, matmul_quantized_with_scratch, src/engine/kernels/quant.rs:7225; batched rows in
// transformer_prefill_batch). With the weights resident on the device only the hidden-state rows cross PCIe.
//
// Two kernels:
//   proj_gemv_kernel  decode, a few activation rows: bound by reading the weights once. One warp per two weight
//                     rows, 16-byte loads along the row, the activation rows come from L1, shuffle reduction.
//                     Weight formats F32, BF16, Q8_0 (codes and f16 block scales repacked into two planes at
//                     upload, so that the codes are 16-byte aligned) and Q4_K (nibble plane in which the 32 weights
//                     of a (scale, min) pair are one 16-byte load; w = d * scale * q - dmin * min is applied as
//                     d * scale * sum(x q) - dmin * min * sum(x), one FMA per weight) and Q6_K (kept as int8 codes
//                     q - 32 with one f32 scale per 16 weights, which is one lane's load).
//   proj_gemm_kernel  prefill chunks: tcgen05 GEMM, bf16 x bf16 -> f32 in TMEM. A = activations [m][K] (bf16), B =
//                     weights [N][K] (bf16; Q8_0 / F32 weights use a bf16 image made at upload), 128 x 256 output
//                     tile per CTA, 64-column k-steps through a four-stage TMA ring, one MMA issuer, four epilogue
//                     warps reading the accumulator out of TMEM. Every wait is bounded.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_utils.cuh"

namespace ggr {

enum ProjWeightType : int { PW_F32 = 0, PW_BF16 = 1, PW_Q8_0 = 2, PW_Q4_K = 3, PW_Q6_K = 4 };

struct GemvArgs {
    const void* w;         // F32 / BF16 values [rows][cols], Q8_0 codes int8 [rows][cols], or Q4_K nibbles [rows][cols / 2]
    const __half* scales;  // Q8_0: f16 scale [rows][cols / 32]; Q4_K: (6-bit scale, 6-bit min) byte pair [rows][cols / 32]
    const __half2* dm;     // Q4_K: (d, dmin) [rows][cols / 256]
    const float* scales_f32;  // Q6_K (codes q - 32 as int8 in w): d * scale per 16 weights [rows][cols / 16]
    int rows, cols;
    const float* x;        // [n][cols]
    int n;
    float* out;            // [n][ld_out]
    int ld_out;
    int sanitize;          // non-finite results become 0 (sanitize_finite_inplace after the output projection)
    // Up to two more matrices of the same type and column count multiplied with the same rows in the same launch (the
    // k and v projections behind the q projection): their rows continue the row numbering of the first matrix.
    // `rows` stays the row count of the first matrix, rows_all is the total.
    int n_extra, rows_all;
    const void* w_x[2];
    const __half* scales_x[2];
    const __half2* dm_x[2];
    const float* scales_f32_x[2];
    int rows_x[2];
    float* out_x[2];
    int ld_out_x[2];
};

// the matrix a (global) row belongs to: its planes, its output and the row's index inside it
struct GemvRowRef {
    const void* w;
    const __half* scales;
    const __half2* dm;
    const float* scales_f32;
    float* out;
    int ld_out, row;
};
__device__ __forceinline__ GemvRowRef gemv_row_ref(const GemvArgs& a, int row) {
    GemvRowRef r{a.w, a.scales, a.dm, a.scales_f32, a.out, a.ld_out, row};
    if (a.n_extra > 0 && row >= a.rows) {
        const bool second = a.n_extra > 1 && row >= a.rows + a.rows_x[0];
        const int i = second ? 1 : 0;  // (selects, not indexed parameter loads)
        r.w = second ? a.w_x[1] : a.w_x[0];
        r.scales = second ? a.scales_x[1] : a.scales_x[0];
        r.dm = second ? a.dm_x[1] : a.dm_x[0];
        r.scales_f32 = second ? a.scales_f32_x[1] : a.scales_f32_x[0];
        r.out = second ? a.out_x[1] : a.out_x[0];
        r.ld_out = second ? a.ld_out_x[1] : a.ld_out_x[0];
        r.row = row - a.rows - (i ? a.rows_x[0] : 0);
    }
    return r;
}

constexpr int kGemvWarps = 8;
constexpr int kGemvRPW = 2;  // weight rows per warp

// 16 bytes of weights, read once: kept out of L1 so that the activation rows (re-read by every warp) stay there
__device__ __forceinline__ uint4 ld_weights16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// int8 code -> float without the conversion unit: the byte, biased by 128, becomes the low mantissa bits of 2^23
// (one byte permute), and subtracting 2^23 + 128 leaves the signed value exactly.
__device__ __forceinline__ float q8_byte_to_float(uint32_t biased_word, int byte) {
    const uint32_t sel = 0x7650u | (uint32_t)byte;  // result bytes: [b, 0x00, 0x00, 0x4B]
    return __uint_as_float(__byte_perm(biased_word, 0x4B000000u, sel)) - 8388736.0f;
}

// byte `byte` of a word as the low mantissa bits of 2^23: the float 8388608 + b (the caller subtracts)
__device__ __forceinline__ float byte_in_mantissa(uint32_t word, int byte) {
    const uint32_t sel = 0x7650u | (uint32_t)byte;  // result bytes: [b, 0x00, 0x00, 0x4B]
    return __uint_as_float(__byte_perm(word, 0x4B000000u, sel));
}

// unsigned byte (0..255) of a word -> float the same way, without a bias
__device__ __forceinline__ float nibble_byte_to_float(uint32_t word, int byte) {
    const uint32_t sel = 0x7650u | (uint32_t)byte;
    return __uint_as_float(__byte_perm(word, 0x4B000000u, sel)) - 8388608.0f;
}

template <int CPL>
__host__ __device__ inline size_t gemv_row_floats_dev(int cols) {
    const int per_step = 32 * CPL;
    return (size_t)((cols + per_step - 1) / per_step) * per_step;
}

template <int WT>
struct GemvGeom {
    static constexpr int CPL = WT == PW_Q4_K ? 32 : ((WT == PW_Q8_0 || WT == PW_Q6_K) ? 16 : 8);  // columns per lane and step (one 16-byte load; two for F32)
    // steps per batch of weight loads; two batches are in flight: the next one is requested before the current one is
    // multiplied, so the memory pipe never waits for the arithmetic
    static constexpr int UN = (WT == PW_F32 || WT == PW_Q4_K) ? 2 : 4;
    static constexpr int SPAN = 32 * CPL * UN;           // columns one batch of loads covers
    static constexpr int NL = WT == PW_F32 ? 2 : 1;      // 16-byte loads per lane, step and row
};

// floats of shared memory one staged activation row takes: whole steps of 32 lanes x CPL columns
template <int WT>
inline size_t gemv_row_floats(int cols) {
    const int per_step = 32 * GemvGeom<WT>::CPL;
    return (size_t)((cols + per_step - 1) / per_step) * per_step;
}

template <int WT, int TT>
// (two CTAs per SM, i.e. at most 128 registers, wherever that needs no spills: one activation row, or unquantised weights;
// the quantised types with several rows need the registers for their decoded weights and accumulators)
__global__ void __launch_bounds__(kGemvWarps * 32, (TT == 1 || WT == PW_F32 || WT == PW_BF16) ? 2 : 1) proj_gemv_kernel(GemvArgs a) {
    using Ge = GemvGeom<WT>;
    constexpr int CPL = Ge::CPL, UN = Ge::UN, NL = Ge::NL, Q = CPL / 4;
    extern __shared__ __align__(16) float xs[];  // [TT][row_floats]: the activation rows of the pass, read by every warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cols = a.cols;
    const int rows_all = a.n_extra > 0 ? a.rows_all : a.rows;
    const int n_groups = (rows_all + kGemvWarps * kGemvRPW - 1) / (kGemvWarps * kGemvRPW);
    const int ncb = (cols + Ge::SPAN - 1) / Ge::SPAN;                       // load batches per row
    const int my_groups = n_groups > (int)blockIdx.x ? (n_groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int n_units = my_groups * ncb;                                    // (row group, batch) units of this CTA
    const int row4 = (int)(gemv_row_floats_dev<CPL>(cols) >> 2);            // float4 pieces per staged row

    struct Batch {
        uint4 raw[UN][kGemvRPW][NL];
        float dsc[UN][kGemvRPW];
        float dmn[UN][kGemvRPW];  // Q4_K: dmin * min of the lane's 32 weights
    };
    Batch ba, bb;
    // requests the weights of unit u: UN steps of both rows, independent 16-byte loads
    auto load_unit = [&](int u, Batch& b) {
        auto& raw = b.raw;
        auto& dsc = b.dsc;
        auto& dmn = b.dmn;
        const int grp = blockIdx.x + (u / ncb) * gridDim.x, cb = (u % ncb) * Ge::SPAN;
        const int r0 = (grp * kGemvWarps + warp) * kGemvRPW;
#pragma unroll
        for (int s = 0; s < UN; ++s) {
            const int c0 = cb + s * 32 * CPL + lane * CPL;
#pragma unroll
            for (int r = 0; r < kGemvRPW; ++r) {
                const GemvRowRef rr = gemv_row_ref(a, min(r0 + r, rows_all - 1));
                const int row = rr.row;
                dsc[s][r] = 1.0f;
                if (c0 < cols) {
                    if (WT == PW_F32) {
                        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(rr.w) + (size_t)row * cols + c0);
                        raw[s][r][0] = ld_weights16(p);
                        raw[s][r][NL - 1] = ld_weights16(p + 1);
                    } else if (WT == PW_BF16) {
                        raw[s][r][0] = ld_weights16(static_cast<const __nv_bfloat16*>(rr.w) + (size_t)row * cols + c0);
                    } else if (WT == PW_Q8_0) {
                        raw[s][r][0] = ld_weights16(static_cast<const int8_t*>(rr.w) + (size_t)row * cols + c0);
                        dsc[s][r] = __half2float(rr.scales[(size_t)row * (cols >> 5) + (c0 >> 5)]);
                    } else if (WT == PW_Q6_K) {
                        // a lane's 16 codes are exactly the weights of one scale
                        raw[s][r][0] = ld_weights16(static_cast<const int8_t*>(rr.w) + (size_t)row * cols + c0);
                        dsc[s][r] = __ldg(rr.scales_f32 + (size_t)row * (cols >> 4) + (c0 >> 4));
                    } else {
                        raw[s][r][0] = ld_weights16(static_cast<const uint8_t*>(rr.w) + (((size_t)row * cols + c0) >> 1));
                        const uint32_t sm = __ldg(reinterpret_cast<const unsigned short*>(rr.scales) + (size_t)row * (cols >> 5) + (c0 >> 5));
                        const float2 dd = __half22float2(__ldg(rr.dm + (size_t)row * (cols >> 8) + (c0 >> 8)));
                        dsc[s][r] = dd.x * (float)(sm & 0xffu);   // d * scale, as dequantize_row_q4_k forms it
                        dmn[s][r] = dd.y * (float)(sm >> 8);      // dmin * min
                    }
                }
            }
        }
    };

    for (int t0 = 0; t0 < a.n; t0 += TT) {
        // the first unit's weights are requested before the activation rows are staged: both latencies overlap
        if (n_units > 0) load_unit(0, ba);
        __syncthreads();  // every warp is done with the rows of the previous pass
        // A lane multiplies CPL consecutive columns per step, i.e. CPL / 4 float4 pieces that lie 4 * CPL bytes apart
        // from its neighbour's: read straight, that is a 4-way (Q8_0) or 2-way bank conflict on every load. The rows
        // are therefore stored piece-major: piece q of step s of all 32 lanes is contiguous.
        const int c4n = cols >> 2;
        for (int i4 = threadIdx.x; i4 < TT * c4n; i4 += kGemvWarps * 32) {
            const int t = i4 / c4n, col4 = i4 - t * c4n;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (t0 + t < a.n) v = __ldg(reinterpret_cast<const float4*>(a.x + (size_t)(t0 + t) * cols) + col4);
            const int step = col4 / (32 * Q), ln = (col4 % (32 * Q)) / Q, q = col4 % Q;
            reinterpret_cast<float4*>(xs)[(size_t)t * row4 + (step * Q + q) * 32 + ln] = v;
        }
        __syncthreads();
        float acc[kGemvRPW][TT];
        // multiplies unit u (its weights are in `b`) into the accumulators; the last unit of a row group stores
        auto compute_unit = [&](int u, const Batch& b) {
            const auto& raw = b.raw;
            const auto& dsc = b.dsc;
            const auto& dmn = b.dmn;
            (void)dmn;
            const int grp = blockIdx.x + (u / ncb) * gridDim.x, cbi = u % ncb, cb = cbi * Ge::SPAN;
            const int r0 = (grp * kGemvWarps + warp) * kGemvRPW;
            if (cbi == 0) {
#pragma unroll
                for (int r = 0; r < kGemvRPW; ++r)
#pragma unroll
                    for (int t = 0; t < TT; ++t) acc[r][t] = 0.0f;
            }
#pragma unroll
            for (int s = 0; s < UN; ++s) {
                const int c0 = cb + s * 32 * CPL + lane * CPL;
                if (c0 >= cols) continue;
                // decoded weights as packed pairs: the arithmetic below handles two weights per instruction
                // (add.f32x2 / fma.rn.f32x2), which is what the kernel is bound by
                using tc::add_f32x2;
                using tc::fma_f32x2;
                using tc::pack_f32x2;
                uint64_t w2[kGemvRPW][CPL / 2];
#pragma unroll
                for (int r = 0; r < kGemvRPW; ++r) {
                    if (WT == PW_F32) {
                        const uint4 u0 = raw[s][r][0], u1 = raw[s][r][NL - 1];
                        w2[r][0] = pack_f32x2(__uint_as_float(u0.x), __uint_as_float(u0.y));
                        w2[r][1] = pack_f32x2(__uint_as_float(u0.z), __uint_as_float(u0.w));
                        w2[r][2 % (CPL / 2)] = pack_f32x2(__uint_as_float(u1.x), __uint_as_float(u1.y));
                        w2[r][3 % (CPL / 2)] = pack_f32x2(__uint_as_float(u1.z), __uint_as_float(u1.w));
                    } else if (WT == PW_BF16) {
                        const uint4 q = raw[s][r][0];
                        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w2[r][i] = pack_f32x2(__uint_as_float(w4[i] << 16), __uint_as_float(w4[i] & 0xffff0000u));
                    } else if (WT == PW_Q8_0 || WT == PW_Q6_K) {
                        // code byte, biased by 128, in the low mantissa bits of 2^23; the bias leaves in one packed add
                        const uint4 q = raw[s][r][0];
                        const uint32_t w4[4] = {q.x ^ 0x80808080u, q.y ^ 0x80808080u, q.z ^ 0x80808080u, q.w ^ 0x80808080u};
                        const uint64_t neg = pack_f32x2(-8388736.0f, -8388736.0f);
#pragma unroll
                        for (int i = 0; i < CPL; i += 2)
                            w2[r][i >> 1] = add_f32x2(pack_f32x2(byte_in_mantissa(w4[(i >> 2) & 3], i & 3),
                                                                 byte_in_mantissa(w4[(i >> 2) & 3], (i & 3) + 1)), neg);
                    } else {
                        // byte i of the 16 holds weights i (low nibble) and i + 16 (high nibble) of the lane's 32
                        const uint4 q = raw[s][r][0];
                        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
                        const uint64_t neg = pack_f32x2(-8388608.0f, -8388608.0f);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t lo = w4[k] & 0x0f0f0f0fu, hi = (w4[k] >> 4) & 0x0f0f0f0fu;
#pragma unroll
                            for (int b = 0; b < 4; b += 2) {
                                w2[r][((4 * k + b) >> 1) % (CPL / 2)] =
                                    add_f32x2(pack_f32x2(byte_in_mantissa(lo, b), byte_in_mantissa(lo, b + 1)), neg);
                                w2[r][((16 + 4 * k + b) >> 1) % (CPL / 2)] =
                                    add_f32x2(pack_f32x2(byte_in_mantissa(hi, b), byte_in_mantissa(hi, b + 1)), neg);
                            }
                        }
                    }
                }
                const int step = (cb + s * 32 * CPL) / (32 * CPL);
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    const float4* xp = reinterpret_cast<const float4*>(xs) + (size_t)t * row4 + (size_t)step * Q * 32 + lane;
                    float part[kGemvRPW];
                    uint64_t pacc[kGemvRPW];  // (even, odd) sums
#pragma unroll
                    for (int r = 0; r < kGemvRPW; ++r) pacc[r] = 0ull;
#pragma unroll
                    for (int i = 0; i < CPL; i += 4) {
                        const float4 xx = xp[(i >> 2) * 32];
                        const uint64_t x01 = pack_f32x2(xx.x, xx.y), x23 = pack_f32x2(xx.z, xx.w);
#pragma unroll
                        for (int r = 0; r < kGemvRPW; ++r) {
                            pacc[r] = fma_f32x2(x01, w2[r][i >> 1], pacc[r]);
                            pacc[r] = fma_f32x2(x23, w2[r][(i >> 1) + 1], pacc[r]);
                        }
                    }
#pragma unroll
                    for (int r = 0; r < kGemvRPW; ++r) {
                        float lo, hi;
                        tc::unpack_f32x2(pacc[r], lo, hi);
                        part[r] = lo + hi;
                    }
                    // Q8_0: the block scale multiplies the partial sum of the block's codes, as in the reference
#pragma unroll
                    for (int r = 0; r < kGemvRPW; ++r) acc[r][t] = fmaf(part[r], dsc[s][r], acc[r][t]);
                    if (WT == PW_Q4_K) {
                        // sum over the lane's 32 weights of x (d s q - dmin m) = d s sum(x q) - dmin m sum(x)
                        float xsum = 0.0f;
#pragma unroll
                        for (int i = 0; i < CPL; i += 4) {
                            const float4 xx = xp[(i >> 2) * 32];
                            xsum += (xx.x + xx.y) + (xx.z + xx.w);
                        }
#pragma unroll
                        for (int r = 0; r < kGemvRPW; ++r) acc[r][t] = fmaf(-dmn[s][r], xsum, acc[r][t]);
                    }
                }
            }
            if (cbi == ncb - 1) {
#pragma unroll
                for (int r = 0; r < kGemvRPW; ++r)
#pragma unroll
                    for (int t = 0; t < TT; ++t) {
                        float v = warp_sum(acc[r][t]);
                        if (lane == 0 && r0 + r < rows_all && t0 + t < a.n) {
                            if (a.sanitize && !isfinite(v)) v = 0.0f;
                            const GemvRowRef rr = gemv_row_ref(a, r0 + r);
                            rr.out[(size_t)(t0 + t) * rr.ld_out + rr.row] = v;
                        }
                    }
            }
        };
        for (int u = 0; u < n_units; u += 2) {
            if (u + 1 < n_units) load_unit(u + 1, bb);
            compute_unit(u, ba);
            if (u + 1 < n_units) {
                if (u + 2 < n_units) load_unit(u + 2, ba);
                compute_unit(u + 1, bb);
            }
        }
    }
}

constexpr int kGemvMaxCols = 12288;  // activation rows are staged in shared memory: up to 48 KB per row

template <int WT, int TT>
inline cudaError_t launch_gemv_inst(const GemvArgs& a, int device, int sm_count, cudaStream_t stream) {
    static KernelSmemSetup setup;
    const size_t smem = (size_t)TT * gemv_row_floats<WT>(a.cols) * sizeof(float);
    cudaError_t e = setup.ensure(proj_gemv_kernel<WT, TT>, device, 0, (int)((size_t)TT * gemv_row_floats<WT>(kGemvMaxCols) * sizeof(float)));
    if (e != cudaSuccess) return e;
    const int groups = ((a.n_extra > 0 ? a.rows_all : a.rows) + kGemvWarps * kGemvRPW - 1) / (kGemvWarps * kGemvRPW);
    // row groups are dealt round robin to a grid that fills the SMs about twice (the staged rows are loaded once per CTA)
    const int grid = groups < 2 * sm_count ? groups : 2 * sm_count;
    proj_gemv_kernel<WT, TT><<<grid, kGemvWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int WT>
inline cudaError_t launch_gemv_wt(const GemvArgs& a, int device, int sm_count, cudaStream_t stream) {
    if (a.n == 1) return launch_gemv_inst<WT, 1>(a, device, sm_count, stream);
    if (a.n == 2) return launch_gemv_inst<WT, 2>(a, device, sm_count, stream);
    return launch_gemv_inst<WT, 4>(a, device, sm_count, stream);
}

inline cudaError_t launch_gemv(int wtype, const GemvArgs& a, int device, int sm_count, cudaStream_t stream) {
    switch (wtype) {
        case PW_F32: return launch_gemv_wt<PW_F32>(a, device, sm_count, stream);
        case PW_BF16: return launch_gemv_wt<PW_BF16>(a, device, sm_count, stream);
        case PW_Q4_K: return launch_gemv_wt<PW_Q4_K>(a, device, sm_count, stream);
        case PW_Q6_K: return launch_gemv_wt<PW_Q6_K>(a, device, sm_count, stream);
        default: return launch_gemv_wt<PW_Q8_0>(a, device, sm_count, stream);
    }
}

// f32 rows -> bf16 rows (activations on their way into the tensor-core GEMM)
__global__ void proj_to_bf16_kernel(const float* src, __nv_bfloat16* dst, size_t n) {
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        if (i + 4 <= n) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t*>(&a);
            u.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>(dst + i) = u;
        } else {
            for (size_t j = i; j < n; ++j) dst[j] = __float2bfloat16_rn(src[j]);
        }
    }
}

// ---- tcgen05 GEMM ------------------------------------------------------------------------------------------

struct GemmArgs {
    int m, N, K;
    float* out;             // [m][ld_out] f32, or null
    __nv_bfloat16* out_h;   // [m][ld_out] bf16, or null
    int ld_out;
    int sanitize;
    int* err;               // raised when a bounded wait runs out
};

constexpr int kGemmBM = 128, kGemmBN = 256, kGemmBK = 64, kGemmStages = 4;
constexpr int kGemmThreads = 192;  // four epilogue warps, a TMA producer, an MMA issuer
constexpr uint32_t kGemmABytes = kGemmBM * kGemmBK * 2, kGemmBBytes = kGemmBN * kGemmBK * 2;
inline size_t proj_gemm_smem() { return (size_t)kGemmStages * (kGemmABytes + kGemmBBytes) + 1024; }

__global__ void __launch_bounds__(kGemmThreads, 1)
proj_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs a) {
    using namespace tc;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kGemmStages + 1];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = smem_base, sB = smem_base + kGemmStages * kGemmABytes;
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kGemmStages + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * kGemmStages);

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&s_tmem_base), kGemmBN);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = s_tmem_base;
    volatile int* abortp = &s_abort;
    const int n0 = blockIdx.x * kGemmBN, m0 = blockIdx.y * kGemmBM;
    const int nk = (a.K + kGemmBK - 1) / kGemmBK;

    if (warp == 4) {
        if (lane == 0) {
            for (int k = 0; k < nk; ++k) {
                const int s = k % kGemmStages;
                if (!mbar_wait(empty(s), ((k / kGemmStages) & 1) ^ 1, abortp)) break;
                mbar_expect_tx(full(s), kGemmABytes + kGemmBBytes);
                tma_load_2d(sA + s * kGemmABytes, &tmA, k * kGemmBK, m0, full(s));
                tma_load_2d(sB + s * kGemmBBytes, &tmB, k * kGemmBK, n0, full(s));
            }
        }
    } else if (warp == 5) {
        constexpr uint32_t IDESC = idesc_bf16(kGemmBN, 0);
        const uint64_t dA = smem_desc(sA, 16, 1024), dB = smem_desc(sB, 16, 1024);
        const uint32_t tm = __shfl_sync(0xffffffffu, s_tmem_base, 0);
        bool ok = true;
        for (int k = 0; k < nk && ok; ++k) {
            const int s = k % kGemmStages;
            if (!(ok = mbar_wait_warp(full(s), (k / kGemmStages) & 1, abortp))) break;
            fence_after_sync();
            const uint64_t a0 = dA + (uint64_t)((s * kGemmABytes) >> 4), b0 = dB + (uint64_t)((s * kGemmBBytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < kGemmBK / 16; ++ks)
                mma_ss_e(tm, a0 + (uint64_t)((ks * 32) >> 4), b0 + (uint64_t)((ks * 32) >> 4), IDESC, (k > 0 || ks > 0) ? 1u : 0u);
            mma_commit_e(empty(s));
        }
        if (ok) mma_commit_e(acc_full);
    } else {
        // epilogue: thread = output row of the tile (TMEM lane), 32 columns per tcgen05.ld
        const int row = m0 + warp * 32 + lane;
        if (mbar_wait(acc_full, 0, abortp)) {
            fence_after_sync();
            const uint32_t t0 = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < kGemmBN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(t0 + c * 32, v);
                tmem_wait_ld();
                const int col0 = n0 + c * 32;
                if (row < a.m && col0 < a.N) {
                    const int ncol = min(32, a.N - col0);
                    if (a.out) {
                        float* o = a.out + (size_t)row * a.ld_out + col0;
                        for (int i = 0; i < ncol; i += 4) {
                            float4 f = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                                                   __uint_as_float(v[i + 3]));
                            if (a.sanitize) {
                                f.x = isfinite(f.x) ? f.x : 0.0f;
                                f.y = isfinite(f.y) ? f.y : 0.0f;
                                f.z = isfinite(f.z) ? f.z : 0.0f;
                                f.w = isfinite(f.w) ? f.w : 0.0f;
                            }
                            *reinterpret_cast<float4*>(o + i) = f;
                        }
                    }
                    if (a.out_h) {
                        __nv_bfloat16* o = a.out_h + (size_t)row * a.ld_out + col0;
                        for (int i = 0; i < ncol; i += 2) {
                            __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                            *reinterpret_cast<__nv_bfloat162*>(o + i) = p;
                        }
                    }
                }
            }
        }
    }
    if (s_abort) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 5) tmem_dealloc(tmem, kGemmBN);
    if (tid == 0 && s_abort && a.err) atomicExch(a.err, 1);
}

// tmA: activations [m][K] with a 64 x 128 box; tmB: weights [N][K] with a 64 x 256 box
inline cudaError_t launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, int device,
                               cudaStream_t stream) {
    static KernelSmemSetup setup;
    const size_t smem = proj_gemm_smem();
    cudaError_t e = setup.ensure(proj_gemm_kernel, device, 0, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((a.N + kGemmBN - 1) / kGemmBN, (a.m + kGemmBM - 1) / kGemmBM);
    proj_gemm_kernel<<<grid, kGemmThreads, smem, stream>>>(tmA, tmB, a);
    return cudaGetLastError();
}

}  // namespace ggr
