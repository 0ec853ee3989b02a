// Shared device-side types of the attention path: the KV-cache view, the item
// table (which cache row each launched item stands for), RoPE parameters and
// small helpers. Everything here is plain data passed by value to kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace ggr {

// Raises a kernel's dynamic shared-memory limit once per device. Contexts are independent and may be
// driven from different host threads, so the bookkeeping is one atomic bit per device ordinal with a
// mutex around the slow path. Each launch helper keeps one (function-local static) per kernel instance.
struct KernelSmemSetup {
    std::atomic<uint64_t> done{0};
    std::mutex mu;

    // bytes < 0 selects the device's opt-in maximum minus the kernel's static shared memory
    template <typename K>
    cudaError_t ensure(K kernel, int device, int smem_optin, int bytes = -1) {
        const bool tracked = device >= 0 && device < 64;
        if (tracked && (done.load(std::memory_order_acquire) >> device) & 1ull) return cudaSuccess;
        std::lock_guard<std::mutex> lock(mu);
        if (tracked && (done.load(std::memory_order_relaxed) >> device) & 1ull) return cudaSuccess;
        int want = bytes;
        if (want < 0) {
            cudaFuncAttributes fa;
            cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
            if (e != cudaSuccess) return e;
            want = smem_optin - (int)fa.sharedSizeBytes;
        }
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, want);
        if (e != cudaSuccess) return e;
        // these kernels stage everything in shared memory: ask for the largest carve-out, so that as many CTAs
        // as the kernel's own footprint allows are resident (the default left one where two fit)
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        if (tracked) done.fetch_or(1ull << device, std::memory_order_release);
        return cudaSuccess;
    }
};

enum KvFormat : int { KV_F32 = 0, KV_BF16 = 1, KV_Q8_ROW = 2, KV_Q8_BLOCK32 = 3, KV_TURBO = 4 };

constexpr int kMaxArgItems = 128;  // positions carried inside the kernel arguments
constexpr float kLog2e = 1.4426950408889634f;

// Device KV cache of one context. Row r = (seq * n_layers + layer) * rows + (pos - pos_begin);
// element r * kv_dim + kv_head * D + i  (the reference's slot layout,
// src/engine/runtime/inference.rs:1880-1882, with a sequence index in front).
struct KvView {
    void* k;
    void* v;
    float* ks;  // q8 scales: one per row (Q8_ROW) or kv_dim/32 per row (Q8_BLOCK32); TurboQuant: sigma per (row, kv head)
    float* vs;
    // TurboQuant only (k / v then hold the packed 2-bit codes): residual sign bits, residual norms per
    // (row, kv head), and the sign tables of the four transforms [slot][layer][kv_head][D / 8]
    unsigned char* k_sign;
    unsigned char* v_sign;
    float* k_rn;
    float* v_rn;
    const unsigned char* turbo_signs;
    int fmt;
    int D, kv_dim, Hkv, Hq, G;
    int n_layers;
    int rows;       // positions held per (sequence, layer)
    int pos_begin;  // first global position held (KV-sequence sharding), else 0
    int elem_bytes;
    int n_scales;  // scales per row: 0, 1 or kv_dim/32

    __host__ __device__ int64_t row(int seq, int layer, int pos) const {
        return ((int64_t)seq * n_layers + layer) * (int64_t)rows + (int64_t)(pos - pos_begin);
    }
};

// Which (sequence, position) an item of a launch stands for.
struct Items {
    int mode;  // 0: decode, item b -> (seq b, pos[b]); 1: prefill, item i -> (seq0, base_pos + i)
    int seq0, base_pos, n;
    int pos[kMaxArgItems];

    __device__ __forceinline__ void get(int item, int& seq, int& p) const {
        if (mode == 0) {
            seq = seq0 + item;
            p = pos[item];
        } else {
            seq = seq0;
            p = base_pos + item;
        }
    }
};

// Mask settings of one layer (src/engine/runtime/attention.rs:73-97).
struct Visibility {
    int window;      // 0 = global
    int image_mode;  // 1 = bidirectional image blocks
    const int2* blocks;  // (token_start, token_len), ordered and disjoint
    int n_blocks;

    __device__ __forceinline__ void range(int pos, int& vs, int& ve) const {
        ve = pos + 1;
        vs = window > 0 ? max(0, ve - window) : 0;
        if (image_mode == 1) {
            for (int i = 0; i < n_blocks; ++i) {
                int2 b = blocks[i];
                if (pos >= b.x && pos - b.x < b.y) {
                    vs = min(vs, b.x);
                    ve = b.x + b.y;
                    break;
                }
            }
        }
    }
};

// RoPE parameters of one layer kind (src/engine/runtime/inference.rs:1485-1523).
struct RopeParams {
    const float* freqs;  // rope_half entries, already the table of this layer kind
    float fscale;        // rope_scaling.local on window layers, .global otherwise
    int rope_half, rope_dim;
    int style;   // 0 NeoX, 1 adjacent pairs
    int layout;  // 1 = interleaved T/H/W
    int sections[4];
    const int* plan;  // [plan_len][3] logical coordinates or null
    int plan_len, next_text, has_plan;
    float q_prescale;  // 1/sqrt(D) in q-prescaled mode
    int do_prescale;
};

__device__ __forceinline__ int rope_axis(int layout, int frequency, const int* sections) {
    if (layout == 0) return 0;
    int axis = frequency % 3;
    if (axis != 0 && frequency / 3 < sections[axis]) return axis;
    return 0;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t hi16) { return __uint_as_float(hi16 << 16); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// cp.async of `bytes` in {4, 8, 16}; src_bytes < bytes zero-fills the rest.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

}  // namespace ggr
