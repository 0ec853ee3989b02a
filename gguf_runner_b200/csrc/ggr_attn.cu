// Context, launch logic and C ABI of the attention path (see include/ggr_attn.h).
// There is no CPU fallback: every entry point that computes launches CUDA
// kernels on the context's device or returns an error status.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ggr_attn.h"
#include "attn_mma.cuh"
#include "attn_simt.cuh"
#include "attn_tile.cuh"
#include "attn_turbo.cuh"
#include "attn_turbo_mma.cuh"
#include "common.cuh"
#include "prefill_tc.cuh"
#include "prefill_tc_wide.cuh"
#include "proj.cuh"
#include "rope_append.cuh"

using namespace ggr;

struct ggr_attn_ctx {
    ggr_attn_config cfg;
    std::vector<int32_t> windows;
    int D = 0, kv_dim = 0, q_dim = 0, G = 0, rope_half = 0, rope_dim = 0;
    float attn_scale = 0.f;
    int shard_begin = 0, shard_count = 0;
    int sm_count = 0, smem_optin = 0;
    cudaStream_t stream = nullptr, own_stream = nullptr;
    KvView kv{};
    float* d_freqs = nullptr;
    float* d_freqs_swa = nullptr;
    int* d_plan = nullptr;
    int plan_len = 0, next_text = 0, has_plan = 0;
    int2* d_blocks = nullptr;
    std::vector<int2> blocks;
    // scratch, grown on demand
    float* d_qrot = nullptr;
    __nv_bfloat16* d_qrot_h = nullptr;
    size_t qrot_cap = 0, qrot_h_cap = 0;
    float* d_krot = nullptr;  // rotated keys on their way into a TurboQuant cache
    size_t krot_cap = 0;
    unsigned char* d_turbo_signs = nullptr;
    float* d_part = nullptr;
    size_t part_cap = 0;
    unsigned* d_counters = nullptr;
    size_t counters_cap = 0;
    // staging for host-pointer calls
    unsigned char* d_stage[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};  // q, k, v, out, gate
    size_t stage_cap[5] = {0, 0, 0, 0, 0};
    float* d_gate_f32 = nullptr;  // f32 image of a bf16 gate for the kernels that take f32 gates
    size_t gate_f32_cap = 0;
    // projections: staged hidden rows (in / out), q | k | v rows, attention output rows, bf16 activation rows
    float* d_px = nullptr;
    float* d_pqkv = nullptr;
    float* d_patt = nullptr;
    float* d_pout = nullptr;
    __nv_bfloat16* d_pact = nullptr;
    __nv_bfloat16* d_pqkv_h = nullptr;
    size_t px_cap = 0, pqkv_cap = 0, patt_cap = 0, pout_cap = 0, pact_cap = 0, pqkv_h_cap = 0;
    // pinned host staging of host-pointer decode calls: q | k | v | gate travel as one copy, the output as one
    unsigned char* h_pin = nullptr;
    unsigned char* d_pin_alias = nullptr;  // device address of h_pin (mapped pinned memory), or null
    size_t pin_cap = 0;
    unsigned char* d_pin_in = nullptr;  // device image of the inbound half
    size_t pin_in_cap = 0;
    int reserved_batch = 0;     // decode batch the scratch is reserved for (0 = grow on demand)
    int reserved_splits = 0;    // split-KV factor the reserved partial-state scratch holds per item
    std::string err;
    int64_t launches = 0;
    int last_splits = 0;  // split-KV factor of the most recent attention launch
    // tensor maps over the whole K and V arrays (bf16 caches) for the TMA prefill kernel
    CUtensorMap tmK, tmV;
    bool have_tmaps = false;
    // the same arrays with a 64 x 64 box for the head_dim 256 prefill kernel
    CUtensorMap tmK64, tmV64;
    bool have_tmaps64 = false;
    // the same arrays with a 64 x 16 box for the TMA-fed decode kernel
    CUtensorMap tmK16, tmV16;
    bool have_tmaps16 = false;
    // error word the kernels raise when a bounded wait runs out (mapped pinned host memory)
    int* h_err = nullptr;
    int* d_err = nullptr;
    int* d_sched = nullptr;  // work counters of the persistent prefill kernel (rewound by the kernel itself)
    // per-layer pre-attention fixups (device arrays, null = absent) and their f32 scratch rows
    struct LayerFixups {
        float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;
        float eps = 1e-6f;
        bool any() const { return q_bias || q_norm; }
    };
    std::vector<LayerFixups> fixups;
    float* d_fix[3] = {nullptr, nullptr, nullptr};
    size_t fix_cap[3] = {0, 0, 0};
    // fused exchange of KV-sequence shards: local receive buffer (flags, then two parities of
    // [n_ranks][max_B][Hq][D + 2] floats), the peers' buffers, step counter
    unsigned char* x_local = nullptr;
    unsigned char* x_peer[kMaxPeers] = {};
    bool x_opened[kMaxPeers] = {};
    int x_max_b = 0;
    int x_epoch = 0;
    bool x_connected = false;
    unsigned long long x_wait_ns = 1000000000ull;
    unsigned* d_done = nullptr;
    // copy streams and events of the pipelined host-buffer prefill
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_done;
    // optional per-kernel timing: event pairs per kind (0 attention, 1 rope/append, 2 merge, 3 projection)
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev[4];
    size_t ev_used[4] = {0, 0, 0, 0};
};

// defined in host_plan.cpp
std::vector<unsigned char> ggr_turbo_sign_table(int n_layers, int n_kv_heads, int head_dim);

namespace {

thread_local std::string g_create_err;
#ifdef GGR_TC_TRACE
long long* g_tc_trace = nullptr;
#endif

int fail(ggr_attn_ctx* c, int status, const std::string& msg) {
    if (c) c->err = msg;
    return status;
}

// maps the error word the kernels raise (1 = a bounded wait ran out, 2 = a peer's flag is ahead of this step)
int take_device_error(ggr_attn_ctx* c, const char* what) {
    if (!c->h_err || !*c->h_err) return GGR_OK;
    const int code = *c->h_err;
    *c->h_err = 0;
    if (code == 2)
        return fail(c, GGR_ERR_COMM, "a peer is more than one step ahead of this rank: resynchronise the exchange "
                                     "(ggr_attn_exchange_resync)");
    return fail(c, GGR_ERR_TIMEOUT, what);
}

#define CUDA_TRY(c, expr)                                                                          \
    do {                                                                                           \
        cudaError_t e_ = (expr);                                                                   \
        if (e_ != cudaSuccess)                                                                     \
            return fail(c, GGR_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));      \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && cur != prev) cudaSetDevice(prev);
    }
};

int elem_bytes_of(int fmt) { return fmt == GGR_KV_F32 ? 4 : (fmt == GGR_KV_BF16 ? 2 : 1); }

template <typename T>
int ensure(ggr_attn_ctx* c, T** ptr, size_t* cap, size_t need_elems) {
    if (need_elems <= *cap) return GGR_OK;
    // earlier launches and copies may still use the old buffer
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    if (c->copy_in) CUDA_TRY(c, cudaStreamSynchronize(c->copy_in));
    if (c->copy_out) CUDA_TRY(c, cudaStreamSynchronize(c->copy_out));
    if (*ptr) cudaFree(*ptr);
    *ptr = nullptr;
    *cap = 0;
    size_t want = std::max(need_elems, (size_t)256);
    cudaError_t e = cudaMalloc((void**)ptr, want * sizeof(T));
    if (e != cudaSuccess) return fail(c, GGR_ERR_ALLOC, std::string("scratch allocation failed: ") + cudaGetErrorString(e));
    *cap = want;
    return GGR_OK;
}

// src/engine/runtime/inference.rs:1821-1825
bool is_swa_layer(const ggr_attn_ctx* c, int l) {
    if (c->windows.empty()) return c->cfg.swa_pattern > 0 && (l % c->cfg.swa_pattern < c->cfg.swa_pattern - 1);
    return c->windows[l] != 0;
}

RopeParams rope_params(const ggr_attn_ctx* c, int layer) {
    RopeParams rp{};
    const bool swa = is_swa_layer(c, layer);
    rp.freqs = (c->cfg.swa_theta_on_window_layers && swa) ? c->d_freqs_swa : c->d_freqs;
    rp.fscale = swa ? c->cfg.rope_scale_local : c->cfg.rope_scale_global;
    rp.rope_half = c->rope_half;
    rp.rope_dim = c->rope_dim;
    rp.style = c->cfg.rope_style;
    rp.layout = c->cfg.rope_layout;
    for (int i = 0; i < 4; ++i) rp.sections[i] = c->cfg.rope_sections[i];
    rp.plan = c->d_plan;
    rp.plan_len = c->plan_len;
    rp.next_text = c->next_text;
    rp.has_plan = c->has_plan;
    rp.q_prescale = c->attn_scale;
    rp.do_prescale = c->cfg.scale_mode == GGR_SCALE_Q_PRESCALED;
    return rp;
}

Visibility visibility(const ggr_attn_ctx* c, int layer) {
    Visibility v{};
    v.window = c->windows.empty() ? 0 : c->windows[layer];
    v.image_mode = c->cfg.image_mode;
    v.blocks = c->d_blocks;
    v.n_blocks = (int)c->blocks.size();
    return v;
}

// host copy of Visibility::range (src/engine/runtime/attention.rs:73-97)
void visible_host(const ggr_attn_ctx* c, int layer, int pos, int* vs, int* ve) {
    int e = pos + 1;
    int w = c->windows.empty() ? 0 : c->windows[layer];
    int s = w > 0 ? std::max(0, e - w) : 0;
    if (c->cfg.image_mode == GGR_IMAGE_BIDIRECTIONAL) {
        for (const int2& b : c->blocks) {
            if (pos >= b.x && pos - b.x < b.y) {
                s = std::min(s, b.x);
                e = b.x + b.y;
                break;
            }
        }
    }
    *vs = s;
    *ve = e;
}

// Brackets one launch with events when kernel timing is on.
struct LaunchTimer {
    ggr_attn_ctx* c;
    cudaEvent_t stop = nullptr;
    LaunchTimer(ggr_attn_ctx* ctx, int kind) : c(ctx) {
        if (!c->timing) return;
        auto& pool = c->ev[kind];
        if (c->ev_used[kind] == pool.size()) {
            cudaEvent_t a = nullptr, b = nullptr;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
            pool.emplace_back(a, b);
        }
        auto& pr = pool[c->ev_used[kind]++];
        cudaEventRecord(pr.first, c->stream);
        stop = pr.second;
    }
    ~LaunchTimer() {
        if (stop) cudaEventRecord(stop, c->stream);
    }
};

int ensure_copy_streams(ggr_attn_ctx* c, int n_pieces) {
    if (!c->copy_in) CUDA_TRY(c, cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
    if (!c->copy_out) CUDA_TRY(c, cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
    while ((int)c->ev_in.size() < n_pieces) {
        cudaEvent_t a = nullptr, b = nullptr;
        CUDA_TRY(c, cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        CUDA_TRY(c, cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        c->ev_in.push_back(a);
        c->ev_done.push_back(b);
    }
    return GGR_OK;
}

// Applies the layer's bias / QK-norm fixups to n rows of q/k/v (device memory, element type es bytes)
// and redirects the pointers to the f32 scratch rows. No-op for layers without fixups.
int apply_fixups(ggr_attn_ctx* c, int layer, int n, const void** q, const void** k, const void** v, int* in_bf16) {
    if ((size_t)layer >= c->fixups.size() || !c->fixups[layer].any()) return GGR_OK;
    const auto& f = c->fixups[layer];
    int rc;
    if ((rc = ensure(c, &c->d_fix[0], &c->fix_cap[0], (size_t)n * c->q_dim))) return rc;
    if ((rc = ensure(c, &c->d_fix[1], &c->fix_cap[1], (size_t)n * c->kv_dim))) return rc;
    if ((rc = ensure(c, &c->d_fix[2], &c->fix_cap[2], (size_t)n * c->kv_dim))) return rc;
    FixupArgs a{};
    a.q = *q;
    a.k = *k;
    a.v = *v;
    a.in_bf16 = *in_bf16;
    a.q_bias = f.q_bias;
    a.k_bias = f.k_bias;
    a.v_bias = f.v_bias;
    a.q_norm = f.q_norm;
    a.k_norm = f.k_norm;
    a.eps = f.eps > 0.0f ? f.eps : 1e-5f;  // src/engine/runtime/inference.rs:2539-2543
    a.Hq = c->kv.Hq;
    a.Hkv = c->kv.Hkv;
    a.D = c->D;
    a.q_out = c->d_fix[0];
    a.k_out = c->d_fix[1];
    a.v_out = c->d_fix[2];
    for (int i0 = 0; i0 < n; i0 += 65535) {
        const int cnt = std::min(65535, n - i0);
        FixupArgs b = a;
        const size_t es = *in_bf16 ? 2 : 4;
        b.q = static_cast<const unsigned char*>(a.q) + (size_t)i0 * c->q_dim * es;
        b.k = static_cast<const unsigned char*>(a.k) + (size_t)i0 * c->kv_dim * es;
        b.v = static_cast<const unsigned char*>(a.v) + (size_t)i0 * c->kv_dim * es;
        b.q_out = a.q_out + (size_t)i0 * c->q_dim;
        b.k_out = a.k_out + (size_t)i0 * c->kv_dim;
        b.v_out = a.v_out + (size_t)i0 * c->kv_dim;
        {
            LaunchTimer t(c, 1);
            qkv_fixup_kernel<<<cnt, 256, 0, c->stream>>>(b);
        }
        CUDA_TRY(c, cudaGetLastError());
        c->launches++;
    }
    *q = c->d_fix[0];
    *k = c->d_fix[1];
    *v = c->d_fix[2];
    *in_bf16 = 0;
    return GGR_OK;
}

int check_layer(ggr_attn_ctx* c, int layer) {
    if (layer < 0 || layer >= c->cfg.n_layers) return fail(c, GGR_ERR_RANGE, "layer outside the cache");
    return GGR_OK;
}

// ---- launches ----------------------------------------------------------------------------

int launch_rope_append(ggr_attn_ctx* c, int layer, const Items& items, int flags, int in_bf16, const void* q,
                       const void* k, const void* v, float* q_out, __nv_bfloat16* q_out_h, float* k_out) {
    RopeAppendArgs a{};
    a.rope = rope_params(c, layer);
    a.kv = c->kv;
    a.items = items;
    a.layer = layer;
    a.flags = flags;
    a.in_bf16 = in_bf16;
    a.q = q;
    a.k = k;
    a.v = v;
    a.q_out = q_out;
    a.q_out_h = q_out_h;
    a.k_out = k_out;
    a.shard_count = c->shard_count;
    // TurboQuant: the rope kernel leaves the rotated keys in a scratch buffer and a second kernel quantises
    // them and the values head by head
    const bool turbo = c->kv.fmt == KV_TURBO;
    const bool turbo_append = turbo && (flags & RF_APPEND);
    const float* turbo_k = nullptr;
    bool skip_rope = false;
    if (turbo_append) {
        if (flags == RF_APPEND && !in_bf16) {
            turbo_k = static_cast<const float*>(k);  // already rotated f32 keys: nothing for the rope kernel to do
            skip_rope = true;
        } else {
            int rc = ensure(c, &c->d_krot, &c->krot_cap, (size_t)items.n * c->kv_dim);
            if (rc) return rc;
            a.flags = (flags & ~RF_APPEND) | RF_WRITE_K;
            a.k_out = c->d_krot;
            turbo_k = c->d_krot;
        }
    }
    size_t smem = (size_t)(2 * c->rope_half + 2 * c->kv_dim + 16) * sizeof(float);
    if (smem > 48 * 1024) {
        CUDA_TRY(c, cudaFuncSetAttribute(rope_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    if (!skip_rope) {
        LaunchTimer t(c, 1);
        if (turbo)
            rope_append_kernel<<<items.n, 256, smem, c->stream>>>(a);
        else if (rope_append_fast_ok(a))
            rope_append_bf16_kernel<<<items.n, 256, 0, c->stream>>>(a);
        else if (rope_append_vec_ok(a) && smem + 16 <= 48 * 1024 && in_bf16)
            rope_append_vec_kernel<__nv_bfloat16><<<items.n, 256, smem + 16, c->stream>>>(a);
        else if (rope_append_vec_ok(a) && smem + 16 <= 48 * 1024)
            rope_append_vec_kernel<float><<<items.n, 256, smem + 16, c->stream>>>(a);
        else
            rope_append_kernel<<<items.n, 256, smem, c->stream>>>(a);
    }
    CUDA_TRY(c, cudaGetLastError());
    if (!skip_rope) c->launches++;
    if (turbo_append) {
        TurboAppendArgs t{};
        t.kv = c->kv;
        t.items = items;
        t.layer = layer;
        t.k_rot = turbo_k;
        t.v = v;
        t.v_bf16 = in_bf16;
        t.shard_count = c->shard_count;
        {
            LaunchTimer lt(c, 1);
            turbo_append_kernel<<<dim3(items.n, c->kv.Hkv), 64, (size_t)4 * c->D * sizeof(float), c->stream>>>(t);
        }
        CUDA_TRY(c, cudaGetLastError());
        c->launches++;
    }
    return GGR_OK;
}

struct SimtPlan {
    int nw, nst, stage_bytes, gh;
    size_t smem;
    int ctas_per_sm;
};

SimtPlan simt_plan(const ggr_attn_ctx* c) {
    SimtPlan p{};
    const int rowbytes = c->D * c->kv.elem_bytes;
    const int nsh = c->kv.fmt == KV_Q8_ROW ? 1 : (c->kv.fmt == KV_Q8_BLOCK32 ? c->D / 32 : 0);
    int stage = 2 * kSimtTK * rowbytes + 2 * kSimtTK * nsh * 4;
    stage = (stage + 15) / 16 * 16;
    p.stage_bytes = stage;
    int gh = 1;
    while (gh < c->G && gh < 8) gh <<= 1;
    p.gh = gh;
    const int big = 200 * 1024, small = 100 * 1024;
    int nw = kSimtWarps, nst = 0;
    for (;; nw >>= 1) {
        if (nw * 3 * stage <= small) {
            nst = 3;
            break;
        }
        nst = std::min(4, big / (nw * stage));
        if (nst >= 2 || nw == 1) break;
    }
    if (nst > 4) nst = 4;
    p.nw = nw;
    p.nst = std::max(nst, 2);
    size_t ring = (size_t)p.nw * p.nst * stage;
    size_t merge = (size_t)p.nw * gh * (c->D + 2) * sizeof(float) + 256;
    p.smem = std::max(ring, merge);
    p.ctas_per_sm = std::max(1, std::min(8, (int)((size_t)(c->smem_optin + 1024) / (p.smem + 4096))));
    return p;
}

template <int FMT, int GH, int NST>
int launch_simt_inst(ggr_attn_ctx* c, const AttnArgs& a, dim3 grid, int nw, size_t smem) {
    static KernelSmemSetup setup;
    CUDA_TRY(c, setup.ensure(attn_simt_kernel<FMT, GH, NST>, c->cfg.device, c->smem_optin));
    {
        LaunchTimer t(c, 0);
        attn_simt_kernel<FMT, GH, NST><<<grid, nw * 32, smem, c->stream>>>(a);
    }
    CUDA_TRY(c, cudaGetLastError());
    c->launches++;
    return GGR_OK;
}

template <int FMT, int GH>
int launch_simt_nst(ggr_attn_ctx* c, const AttnArgs& a, dim3 grid, const SimtPlan& p) {
    switch (p.nst) {
        case 2: return launch_simt_inst<FMT, GH, 2>(c, a, grid, p.nw, p.smem);
        case 3: return launch_simt_inst<FMT, GH, 3>(c, a, grid, p.nw, p.smem);
        default: return launch_simt_inst<FMT, GH, 4>(c, a, grid, p.nw, p.smem);
    }
}

template <int FMT>
int launch_simt_gh(ggr_attn_ctx* c, const AttnArgs& a, dim3 grid, const SimtPlan& p) {
    switch (p.gh) {
        case 1: return launch_simt_nst<FMT, 1>(c, a, grid, p);
        case 2: return launch_simt_nst<FMT, 2>(c, a, grid, p);
        case 4: return launch_simt_nst<FMT, 4>(c, a, grid, p);
        default: return launch_simt_nst<FMT, 8>(c, a, grid, p);
    }
}

int launch_simt(ggr_attn_ctx* c, const AttnArgs& a, dim3 grid, const SimtPlan& p) {
    switch (c->kv.fmt) {
        case KV_F32: return launch_simt_gh<KV_F32>(c, a, grid, p);
        case KV_BF16: return launch_simt_gh<KV_BF16>(c, a, grid, p);
        case KV_Q8_ROW: return launch_simt_gh<KV_Q8_ROW>(c, a, grid, p);
        default: return launch_simt_gh<KV_Q8_BLOCK32>(c, a, grid, p);
    }
}

// Split-KV factor. The grid is base_ctas * n CTAs running `slots` at a time, each CTA streaming
// ceil(T / n) keys of `bytes_per_key` bytes. A wave of c concurrent CTAs moves data at
// min(per-CTA rate, HBM rate / c) per CTA and costs a fixed start/finish time; merging n splits
// costs a little per split. The constants are measured on B200 (TMA-fed decode kernel: ~65 GB/s per
// CTA alone, ~6.6 TB/s for the whole GPU, ~8 us per wave). Picks the n with the smallest modelled time.
int choose_splits(int64_t base_ctas, int64_t slots, int t_max, int min_keys, int max_splits, double bytes_per_key,
                  double cta_rate, double t_wave = 8e-6) {
    int limit = std::max(1, t_max / std::max(1, min_keys));
    limit = std::min(limit, 512);
    if (max_splits > 0) limit = std::min(limit, max_splits);
    const double hbm_rate = 6.6e12;
    int best = 1;
    double best_cost = -1.0;
    for (int n = 1; n <= limit; ++n) {
        const int64_t ctas = base_ctas * n;
        const int64_t full = ctas / slots, rem = ctas % slots;
        const double bytes = (double)((t_max + n - 1) / n) * bytes_per_key;
        double cost = 0.0;
        if (full > 0) cost += (double)full * (t_wave + bytes / std::min(cta_rate, hbm_rate / (double)slots));
        if (rem > 0) cost += t_wave + bytes / std::min(cta_rate, hbm_rate / (double)rem);
        // the split merge fetches the states of 16 splits per round trip (~1.4 us each)
        if (n > 1) cost += 2e-6 + 1.4e-6 * ((n + 15) / 16);
        if (best_cost < 0.0 || cost < best_cost) {
            best_cost = cost;
            best = n;
        }
    }
    return best;
}

bool use_mma_decode(const ggr_attn_ctx* c) {
    const bool can = c->kv.fmt == KV_BF16 && mma_decode_supported(c->D, c->G);
    if (c->cfg.decode_impl == GGR_IMPL_MMA) return can;
    if (c->cfg.decode_impl == GGR_IMPL_SIMT) return false;
    return can && c->G >= 3;
}

// shared memory of the split merge: one weight and one l per (head, split), and the sub-results of the warps
// that share a head (only when a CTA has at least twice as many warps as heads, i.e. up to four heads)
size_t split_merge_smem_bytes(const ggr_attn_ctx* c, int n_split) {
    if (n_split <= 1) return 0;
    return ((size_t)2 * c->G * n_split + 2 * c->G + split_merge_sub_floats(c->G, c->D)) * sizeof(float);
}

// Kernel family and launch geometry of a decode / generic attention launch.
struct DecodePlan {
    bool mma, tma, tile;
    SimtPlan p;
    TilePlan tp;
    size_t smem;
    int ctas_per_sm, min_keys;
    double cta_rate;
};

void use_tile_plan(const ggr_attn_ctx* c, DecodePlan& d, int nst) {
    d.tp = tile_plan(c->kv.fmt, c->D, nst, c->smem_optin);
    d.smem = d.tp.smem;
    d.ctas_per_sm = d.tp.ctas_per_sm;
    d.min_keys = d.tp.tk;
    d.cta_rate = 20e9;
}

DecodePlan decode_plan(const ggr_attn_ctx* c, bool allow_mma) {
    DecodePlan d{};
    d.mma = allow_mma && use_mma_decode(c);
    d.tma = d.mma && c->have_tmaps16 && c->cfg.decode_impl != GGR_IMPL_MMA;
    d.p = simt_plan(c);
    d.smem = d.p.smem;
    d.ctas_per_sm = d.p.ctas_per_sm;
    d.min_keys = d.p.nw * kSimtTK * 2;
    d.cta_rate = d.tma ? 65e9 : 40e9;
    if (d.mma) {
        MmaPlan mp = d.tma ? mma_tma_plan(c->D, c->smem_optin) : mma_plan(c->D, c->smem_optin);
        d.smem = mp.smem;
        d.ctas_per_sm = mp.ctas_per_sm;
        d.min_keys = mp.min_keys;
    } else if (allow_mma && c->cfg.decode_impl != GGR_IMPL_SIMT && tile_decode_supported(c->kv.fmt, c->D)) {
        // decode of the formats / groupings the tensor-core kernels do not take: the CTA-tile kernel
        d.tile = true;
        use_tile_plan(c, d, 1);
    }
    return d;
}

// Split-KV factor of a launch. The CTA-tile kernel streams with one ring stage when every CTA gets a single tile
// and with two otherwise, which changes its occupancy and so the split count: settle both here.
int plan_splits(const ggr_attn_ctx* c, DecodePlan& d, int n_items, int t_max, int max_splits) {
    auto pick = [&]() {
        return choose_splits((int64_t)c->kv.Hkv * n_items, (int64_t)c->sm_count * d.ctas_per_sm, t_max, d.min_keys,
                             max_splits, 2.0 * c->D * c->kv.elem_bytes, d.cta_rate, d.tile ? 3e-6 : 8e-6);
    };
    int n = pick();
    if (d.tile && ((t_max + n - 1) / n + d.tp.tk - 1) / d.tp.tk > 1) {
        use_tile_plan(c, d, 2);
        n = pick();
    }
    return n;
}

// Output gate of a call (src/engine/runtime/inference.rs:3509-3519); p == nullptr = none.
struct GateSpec {
    const void* p;
    int head_stride;
    int bf16;
};

// Attention over the cache for `items` (already rotated q at q_dev).
// When `raw` is given (decode), q_dev is scratch for the rotated queries: the kernels rotate q and
// append the k / v row themselves if the fusion scratch fits in shared memory, otherwise the
// rope/append kernel runs first.
struct RawDecodeInputs {
    const float* q;
    const float* k;
    const float* v;
};

int launch_attention(ggr_attn_ctx* c, int layer, const Items& items, int t_max, const float* q_dev, float* out_dev,
                     float* partial_dev, bool allow_mma, const RawDecodeInputs* raw = nullptr,
                     const PeerExchange* px = nullptr, const GateSpec* gate = nullptr) {
    AttnArgs a{};
    a.kv = c->kv;
    a.items = items;
    a.vis = visibility(c, layer);
    a.layer = layer;
    a.q = q_dev;
    a.score_scale = (c->cfg.scale_mode == GGR_SCALE_SCORE ? c->attn_scale : 1.0f) * kLog2e;
    a.out = out_dev;
    a.partial_out = partial_dev;
    a.shard_count = c->shard_count;
    if (px) a.px = *px;
    a.err = c->d_err;
    if (gate && gate->p) {
        a.gate = static_cast<const float*>(gate->p);  // callers hand f32 gates to this path
        a.gate_head_stride = gate->head_stride;
    }

    if (c->kv.fmt == KV_TURBO) {
        // TurboQuant cache: rope + quantising append as separate launches, then the CUDA-core attention kernel.
        // Splits fill the GPU about four CTAs deep (the kernel is bound by arithmetic, not by HBM).
        if (raw) {
            int rc = launch_rope_append(c, layer, items, RF_ROTATE | RF_WRITE_Q | RF_APPEND, 0, raw->q, raw->k, raw->v,
                                        const_cast<float*>(q_dev), nullptr, nullptr);
            if (rc) return rc;
        }
        const int64_t base_ctas = (int64_t)c->kv.Hkv * items.n;
        // tensor-core kernel (head_dim 128, at most 16 query heads per KV head): one 8-warp CTA per SM, splits fill
        // the SMs once; the CUDA-core kernel otherwise (and when decode_impl asks for it): four CTAs per SM deep
        // Prefill rows stay on the f32 CUDA-core kernel unless prefill_impl asks for the tensor-core one
        // (3.5x faster per 512-row chunk at a 3.5 K prefix, bf16-class error instead of 1e-3)
        const bool tc = turbo_mma_supported(c->D, c->G) &&
                        (allow_mma ? c->cfg.decode_impl != GGR_IMPL_SIMT : c->cfg.prefill_impl == GGR_IMPL_MMA);
        const int per_cta_keys = tc ? 2 * kTmWarps * kTmTK : 4 * kTurboGroups;
        int limit = std::min(64, std::max(1, t_max / per_cta_keys));
        if (c->cfg.max_splits > 0) limit = std::min(limit, c->cfg.max_splits);
        int n_split = (int)std::max<int64_t>(1, ((int64_t)4 * c->sm_count + base_ctas - 1) / base_ctas);
        if (tc) {
            // the kernel is bound by its own arithmetic (expanding the codes), so what matters is that the last
            // wave is full: the smallest split count whose CTAs fill at least 95 % of their waves, else the fullest
            double best_eff = -1.0;
            n_split = 1;
            for (int n = 1; n <= limit; ++n) {
                const int64_t ctas = base_ctas * n, waves = (ctas + c->sm_count - 1) / c->sm_count;
                const double eff = (double)ctas / (double)(waves * c->sm_count);
                if (eff > best_eff + 1e-9) {
                    best_eff = eff;
                    n_split = n;
                }
                if (eff >= 0.95) break;
            }
        }
        n_split = std::min(n_split, limit);
        a.n_split = n_split;
        c->last_splits = n_split;
        if (n_split > 1) {
            int rc = ensure(c, &c->d_part, &c->part_cap, (size_t)items.n * c->kv.Hq * n_split * (c->D + 2));
            if (rc) return rc;
            const size_t before = c->counters_cap;
            rc = ensure(c, &c->d_counters, &c->counters_cap, (size_t)items.n * c->kv.Hkv);
            if (rc) return rc;
            if (c->counters_cap != before)
                CUDA_TRY(c, cudaMemsetAsync(c->d_counters, 0, c->counters_cap * sizeof(unsigned), c->stream));
            a.part = c->d_part;
            a.counters = c->d_counters;
        }
        int e;
        if (tc) {
            const size_t smem = turbo_mma_smem_bytes(c->G, n_split);
            a.stage_bytes = (int)turbo_mma_prep_offset(c->G, n_split);
            LaunchTimer t(c, 0);
            e = launch_turbo_mma(a, dim3(n_split, c->kv.Hkv, items.n), smem, c->smem_optin, c->cfg.device, c->stream);
        } else {
            const size_t smem = turbo_attn_smem_floats(c->D, c->G, turbo_heads_per_pass(c->G, c->D), n_split) * sizeof(float);
            if (smem + 1024 > (size_t)c->smem_optin)
                return fail(c, GGR_ERR_UNSUPPORTED, "TurboQuant attention: too many query heads per KV head for shared memory");
            LaunchTimer t(c, 0);
            e = launch_turbo_attention(a, dim3(n_split, c->kv.Hkv, items.n), smem, c->smem_optin, c->cfg.device, c->stream);
        }
        if (e != 0) return fail(c, GGR_ERR_CUDA, std::string("TurboQuant attention launch: ") + cudaGetErrorString((cudaError_t)e));
        c->launches++;
        return GGR_OK;
    }

    DecodePlan dp = decode_plan(c, allow_mma);
    int n_split = plan_splits(c, dp, items.n, t_max, c->cfg.max_splits);
    {
        // with a reservation in place the split count never outgrows the reserved scratch (as long as that
        // holds two splits): the decode loop then neither allocates nor synchronises for memory
        const size_t per_split = (size_t)items.n * c->kv.Hq * (c->D + 2);
        if (c->reserved_batch > 0 && per_split * n_split > c->part_cap) {
            const int fit = (int)std::min<size_t>(512, c->part_cap / per_split);
            if (fit >= 2) n_split = std::min(n_split, fit);
        }
    }
    const bool mma = dp.mma, tma = dp.tma, tile = dp.tile;
    SimtPlan p = dp.p;
    if (tile) p.smem = dp.smem;  // one size governs below: the tile kernel replaces the per-warp-ring kernel
    size_t smem = dp.smem;
    a.stage_bytes = p.stage_bytes;
    a.tile_stages = dp.tp.nst;
    a.err = c->d_err;
    if (raw) {
        const size_t fb = fused_rope_smem_bytes(c->kv, c->rope_half);
        const size_t base = (std::max(smem, p.smem) + 15) & ~(size_t)15;
        // the cp.async-fed tensor-core kernel has no fused prologue; the tile kernel reads the rotated query as
        // 16-byte pieces, which the scratch layout guarantees for an even number of rotated pairs
        const bool kernel_ok = (!mma || tma) && !(tile && (c->rope_half & 1));
        if (c->cfg.decode_fusion == 0 && kernel_ok && base + fb + 4096 <= (size_t)c->smem_optin) {
            a.fused.enabled = 1;
            a.fused.rope = rope_params(c, layer);
            a.fused.q_in = raw->q;
            a.fused.k_in = raw->k;
            a.fused.v_in = raw->v;
            a.fused.smem_off = (int)base;
            smem = base + fb;
            p.smem = base + fb;
        } else {
            int rc = launch_rope_append(c, layer, items, RF_ROTATE | RF_WRITE_Q | RF_APPEND, 0, raw->q, raw->k, raw->v,
                                        const_cast<float*>(q_dev), nullptr, nullptr);
            if (rc) return rc;
        }
    }

    a.n_split = n_split;
    c->last_splits = n_split;
    // the split merge stages one weight per (head, split) in shared memory
    const size_t merge_smem = split_merge_smem_bytes(c, n_split);
    smem = std::max(smem, merge_smem);
    p.smem = std::max(p.smem, merge_smem);
    if (a.fused.enabled && merge_smem > (size_t)a.fused.smem_off) {
        // tiny rings: keep the fusion scratch behind the merge area
        const size_t fb = fused_rope_smem_bytes(c->kv, c->rope_half);
        a.fused.smem_off = (int)((merge_smem + 15) & ~(size_t)15);
        smem = p.smem = (size_t)a.fused.smem_off + fb;
    }
    if (n_split > 1) {
        int rc = ensure(c, &c->d_part, &c->part_cap, (size_t)items.n * c->kv.Hq * n_split * (c->D + 2));
        if (rc) return rc;
        const size_t before = c->counters_cap;
        rc = ensure(c, &c->d_counters, &c->counters_cap, (size_t)items.n * c->kv.Hkv);
        if (rc) return rc;
        if (c->counters_cap != before)
            CUDA_TRY(c, cudaMemsetAsync(c->d_counters, 0, c->counters_cap * sizeof(unsigned), c->stream));
        a.part = c->d_part;
        a.counters = c->d_counters;
    }
    dim3 grid(n_split, c->kv.Hkv, items.n);
#ifdef GGR_TC_TRACE
    a.trace = g_tc_trace;
#endif
    if (mma) {
        int rc;
        {
            LaunchTimer t(c, 0);
            rc = tma ? launch_mma_tma_decode(c->tmK16, c->tmV16, a, grid, smem, c->smem_optin, c->cfg.device, c->stream)
                     : launch_mma_decode(a, grid, smem, c->smem_optin, c->cfg.device, c->stream);
        }
        if (rc != 0) return fail(c, GGR_ERR_CUDA, std::string("mma decode launch: ") + cudaGetErrorString((cudaError_t)rc));
        c->launches++;
        return GGR_OK;
    }
    if (tile) {
        int rc;
        {
            LaunchTimer t(c, 0);
            rc = launch_tile_decode(a, grid, smem, c->smem_optin, c->cfg.device, c->stream);
        }
        if (rc != 0) return fail(c, GGR_ERR_CUDA, std::string("tile decode launch: ") + cudaGetErrorString((cudaError_t)rc));
        c->launches++;
        return GGR_OK;
    }
    return launch_simt(c, a, grid, p);
}

// copies a caller buffer into a staging slot when the caller's memory is host memory
int stage_in(ggr_attn_ctx* c, int slot, const void* src, size_t bytes, int ptr_kind, const void** dev) {
    if (ptr_kind == GGR_PTR_DEVICE) {
        *dev = src;
        return GGR_OK;
    }
    int rc = ensure(c, &c->d_stage[slot], &c->stage_cap[slot], bytes);
    if (rc) return rc;
    CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[slot], src, bytes, cudaMemcpyHostToDevice, c->stream));
    *dev = c->d_stage[slot];
    return GGR_OK;
}

int t_max_of(const ggr_attn_ctx* c, int layer, const int32_t* pos, int n) {
    int t = 1;
    for (int i = 0; i < n; ++i) {
        int vs, ve;
        visible_host(c, layer, pos[i], &vs, &ve);
        vs = std::max(vs, c->shard_begin);
        ve = std::min(ve, c->shard_begin + c->shard_count);
        t = std::max(t, ve - vs);
    }
    return t;
}

// Pinned host staging of host-pointer decode calls: the inbound arrays are packed into one pinned buffer and
// travel in one copy (three pageable copies cost three driver round trips), the result comes back through
// the same buffer. Layout: [in_bytes inbound][out_bytes outbound].
int ensure_pinned(ggr_attn_ctx* c, size_t in_bytes, size_t out_bytes) {
    const size_t need = in_bytes + out_bytes;
    if (need > c->pin_cap) {
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        if (c->h_pin) cudaFreeHost(c->h_pin);
        c->h_pin = nullptr;
        c->pin_cap = 0;
        const size_t want = std::max(need, (size_t)4096);
        if (cudaHostAlloc((void**)&c->h_pin, want, cudaHostAllocMapped) != cudaSuccess) {
            cudaGetLastError();
            return fail(c, GGR_ERR_ALLOC, "unable to allocate pinned staging memory");
        }
        c->pin_cap = want;
        // the device's view of the buffer: decode kernels write their few KB of output straight into it
        void* alias = nullptr;
        if (cudaHostGetDevicePointer(&alias, c->h_pin, 0) != cudaSuccess) {
            cudaGetLastError();
            alias = nullptr;
        }
        c->d_pin_alias = static_cast<unsigned char*>(alias);
    }
    return ensure(c, &c->d_pin_in, &c->pin_in_cap, in_bytes);
}

// outputs up to this size are written by the decode kernels straight into mapped pinned host memory
constexpr size_t kZeroCopyOutBytes = 64 * 1024;

// Sizes of the decode scratch for batches of up to B items (see ggr_attn_reserve).
int reserve_decode(ggr_attn_ctx* c, int B) {
    int rc;
    if ((rc = ensure(c, &c->d_qrot, &c->qrot_cap, (size_t)B * c->q_dim))) return rc;
    int splits = 1;
    if (c->kv.fmt == KV_TURBO) {
        splits = c->cfg.max_splits > 0 ? std::min(64, c->cfg.max_splits) : 64;
        if ((rc = ensure(c, &c->d_krot, &c->krot_cap, (size_t)B * c->kv_dim))) return rc;
    } else {
        // the split count is not monotone in the context length: take the largest over a sweep of lengths
        const int chunk = std::min(B, kMaxArgItems);
        for (int t = c->shard_count; t >= 1; t = t * 3 / 4) {
            DecodePlan dp = decode_plan(c, true);
            splits = std::max(splits, plan_splits(c, dp, chunk, t, c->cfg.max_splits));
            if (t == 1) break;
        }
    }
    const int chunk = std::min(B, kMaxArgItems);
    if (splits > 1) {
        if ((rc = ensure(c, &c->d_part, &c->part_cap, (size_t)chunk * c->kv.Hq * splits * (c->D + 2)))) return rc;
        const size_t before = c->counters_cap;
        if ((rc = ensure(c, &c->d_counters, &c->counters_cap, (size_t)chunk * c->kv.Hkv))) return rc;
        if (c->counters_cap != before)
            CUDA_TRY(c, cudaMemsetAsync(c->d_counters, 0, c->counters_cap * sizeof(unsigned), c->stream));
    }
    // host-pointer calls: q | k | v | gate inbound (a packed gate spans up to 2 * q_dim per token), out or partial outbound
    const size_t in_bytes = ((size_t)B * (c->q_dim + 2 * c->kv_dim) + (size_t)B * 2 * c->q_dim) * sizeof(float);
    const size_t out_bytes = (size_t)B * c->kv.Hq * (c->D + 2) * sizeof(float);
    if ((rc = ensure_pinned(c, in_bytes, out_bytes))) return rc;
    if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], out_bytes))) return rc;
    c->reserved_batch = B;
    c->reserved_splits = splits;
    return GGR_OK;
}

int decode_common(ggr_attn_ctx* c, int layer, const int32_t* pos, int B, const float* q, const float* k,
                  const float* v, float* out, float* partial, int ptr_kind, const float* gate = nullptr,
                  int gate_head_stride = 0) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (B <= 0 || B > c->cfg.max_batch) return fail(c, GGR_ERR_RANGE, "batch larger than max_batch");
    if (!pos || !q || !k || !v || (!out && !partial)) return fail(c, GGR_ERR_INVALID, "null buffer");
    for (int b = 0; b < B; ++b)
        if (pos[b] < 0 || pos[b] >= c->cfg.seq_len) return fail(c, GGR_ERR_RANGE, "position outside the cache");
    if (c->cfg.shard_mode != GGR_SHARD_NONE && !partial)
        return fail(c, GGR_ERR_INVALID, "a KV-sequence shard produces partial states: call ggr_attn_decode_partial");
    if (gate && (partial || gate_head_stride < c->D))
        return fail(c, GGR_ERR_INVALID, "the output gate needs a final output and a head stride of at least head_dim");

    const size_t qb = (size_t)B * c->q_dim * sizeof(float), kb = (size_t)B * c->kv_dim * sizeof(float);
    // elements from the gate pointer to the end of the last head's row
    const size_t gate_elems = gate ? ((size_t)B * c->kv.Hq - 1) * gate_head_stride + c->D : 0;
    const size_t gb = gate_elems * sizeof(float);
    const size_t out_elems = partial ? (size_t)B * c->kv.Hq * (c->D + 2) : (size_t)B * c->q_dim;
    const void *dq = q, *dk = k, *dv = v;
    const float* dgate = gate;
    float* dout = partial ? partial : out;
    bool zero_copy_out = false;
    if (ptr_kind == GGR_PTR_HOST) {
        const size_t in_bytes = qb + 2 * kb + gb;
        if ((rc = ensure_pinned(c, in_bytes, out_elems * sizeof(float)))) return rc;
        if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], out_elems * sizeof(float)))) return rc;
        std::memcpy(c->h_pin, q, qb);
        std::memcpy(c->h_pin + qb, k, kb);
        std::memcpy(c->h_pin + qb + kb, v, kb);
        if (gate) std::memcpy(c->h_pin + qb + 2 * kb, gate, gb);
        CUDA_TRY(c, cudaMemcpyAsync(c->d_pin_in, c->h_pin, in_bytes, cudaMemcpyHostToDevice, c->stream));
        dq = c->d_pin_in;
        dk = c->d_pin_in + qb;
        dv = c->d_pin_in + qb + kb;
        if (gate) dgate = reinterpret_cast<const float*>(c->d_pin_in + qb + 2 * kb);
        dout = reinterpret_cast<float*>(c->d_stage[3]);
        // small outputs (a few rows) go straight into the mapped pinned buffer: one copy and its launch less per call
        if (c->d_pin_alias && out_elems * sizeof(float) <= kZeroCopyOutBytes) {
            const size_t off = c->pin_cap - out_elems * sizeof(float);
            dout = reinterpret_cast<float*>(c->d_pin_alias + off);
            zero_copy_out = true;
        }
    }
    if ((rc = ensure(c, &c->d_qrot, &c->qrot_cap, (size_t)B * c->q_dim))) return rc;
    int in_bf16 = 0;
    if ((rc = apply_fixups(c, layer, B, &dq, &dk, &dv, &in_bf16))) return rc;

    for (int b0 = 0; b0 < B; b0 += kMaxArgItems) {
        const int n = std::min(kMaxArgItems, B - b0);
        Items it{};
        it.mode = 0;
        it.seq0 = b0;
        it.n = n;
        for (int i = 0; i < n; ++i) it.pos[i] = pos[b0 + i];
        const float* qc = reinterpret_cast<const float*>(dq) + (size_t)b0 * c->q_dim;
        const float* kc = reinterpret_cast<const float*>(dk) + (size_t)b0 * c->kv_dim;
        const float* vc = reinterpret_cast<const float*>(dv) + (size_t)b0 * c->kv_dim;
        float* qr = c->d_qrot + (size_t)b0 * c->q_dim;
        const int t_max = t_max_of(c, layer, pos + b0, n);
        float* oc = partial ? nullptr : dout + (size_t)b0 * c->q_dim;
        float* pc = partial ? dout + (size_t)b0 * c->kv.Hq * (c->D + 2) : nullptr;
        const RawDecodeInputs raw{qc, kc, vc};
        GateSpec gs{dgate ? dgate + (size_t)b0 * c->kv.Hq * gate_head_stride : nullptr, gate_head_stride, 0};
        rc = launch_attention(c, layer, it, t_max, qr, oc, pc, true, &raw, nullptr, &gs);
        if (rc) return rc;
    }
    if (ptr_kind == GGR_PTR_HOST) {
        unsigned char* h_out = c->h_pin + (c->pin_cap - out_elems * sizeof(float));
        if (!zero_copy_out)
            CUDA_TRY(c, cudaMemcpyAsync(h_out, dout, out_elems * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        std::memcpy(partial ? partial : out, h_out, out_elems * sizeof(float));
        if (c->h_err && *c->h_err) {
            *c->h_err = 0;
            return fail(c, GGR_ERR_TIMEOUT, "a bounded wait inside the decode kernel ran out");
        }
    }
    return GGR_OK;
}

__global__ void gate_to_f32_kernel(const __nv_bfloat16* src, float* dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __bfloat162float(src[i]);
}

int prefill_common(ggr_attn_ctx* c, int layer, int seq, int base_pos, int m, const void* q, const void* k,
                   const void* v, int in_dtype, float* out, int ptr_kind, bool block_mode, const void* gate = nullptr,
                   int gate_head_stride = 0) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (seq < 0 || seq >= c->cfg.max_batch) return fail(c, GGR_ERR_RANGE, "sequence outside the cache");
    if (m <= 0 || base_pos < 0 || (int64_t)base_pos + m > c->cfg.seq_len)
        return fail(c, GGR_ERR_RANGE, "prefill rows outside the cache");
    if (!q || !k || !v || !out) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (in_dtype != GGR_DTYPE_F32 && in_dtype != GGR_DTYPE_BF16) return fail(c, GGR_ERR_INVALID, "unknown input dtype");
    if (c->cfg.shard_mode != GGR_SHARD_NONE)
        return fail(c, GGR_ERR_UNSUPPORTED, "prefill runs on an unsharded context (shard heads across contexts instead)");
    if (c->cfg.image_mode == GGR_IMAGE_BIDIRECTIONAL) {
        for (const int2& b : c->blocks) {
            const bool overlap = b.x < base_pos + m && base_pos < b.x + b.y;
            if (!block_mode && overlap)
                // src/engine/runtime/inference.rs:2750-2757
                return fail(c, GGR_ERR_INVALID, "batched prefill cannot include complete-block image attention");
            if (block_mode && overlap && (b.x < base_pos || b.x + b.y > base_pos + m))
                return fail(c, GGR_ERR_INVALID, "staged prefill must cover whole image blocks");
        }
    }
    if (gate && gate_head_stride < c->D) return fail(c, GGR_ERR_INVALID, "the gate's head stride must be at least head_dim");
    const size_t es = in_dtype == GGR_DTYPE_BF16 ? 2 : 4;
    const bool host = ptr_kind == GGR_PTR_HOST;
    const unsigned char *dq = static_cast<const unsigned char*>(q), *dk = static_cast<const unsigned char*>(k),
                        *dv = static_cast<const unsigned char*>(v);
    const unsigned char* dgate = static_cast<const unsigned char*>(gate);
    const size_t gate_row = (size_t)c->kv.Hq * gate_head_stride;                     // elements per token
    const size_t gate_elems = gate ? ((size_t)m * c->kv.Hq - 1) * gate_head_stride + c->D : 0;
    float* dout = out;
    if (host && gate) {
        if ((rc = ensure(c, &c->d_stage[4], &c->stage_cap[4], gate_elems * es))) return rc;
        dgate = c->d_stage[4];
    }
    if (host) {
        if ((rc = ensure(c, &c->d_stage[0], &c->stage_cap[0], (size_t)m * c->q_dim * es))) return rc;
        if ((rc = ensure(c, &c->d_stage[1], &c->stage_cap[1], (size_t)m * c->kv_dim * es))) return rc;
        if ((rc = ensure(c, &c->d_stage[2], &c->stage_cap[2], (size_t)m * c->kv_dim * es))) return rc;
        if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], (size_t)m * c->q_dim * sizeof(float)))) return rc;
        dq = c->d_stage[0];
        dk = c->d_stage[1];
        dv = c->d_stage[2];
        dout = reinterpret_cast<float*>(c->d_stage[3]);
    }

    const bool wide = c->have_tmaps64 && c->cfg.prefill_impl != GGR_IMPL_SIMT;
    const bool tc = wide || (c->have_tmaps && prefill_tc_usable(c->cfg.prefill_impl, c->kv.fmt, c->D, c->G));
    if (c->cfg.prefill_impl == GGR_IMPL_TCGEN05 && !tc)
        return fail(c, GGR_ERR_UNSUPPORTED, "the tensor-core prefill kernels need a bf16 cache and head_dim 64, 128 or 256");
    if ((rc = ensure(c, &c->d_qrot, &c->qrot_cap, tc ? (size_t)1 : (size_t)m * c->q_dim))) return rc;
    if (tc && (rc = ensure(c, &c->d_qrot_h, &c->qrot_h_cap, (size_t)m * c->q_dim))) return rc;
    // the CUDA-core kernels take f32 gates: a bf16 gate is widened once the rows are on the device
    const bool widen_gate = gate && !tc && in_dtype == GGR_DTYPE_BF16;
    if (widen_gate && (rc = ensure(c, &c->d_gate_f32, &c->gate_f32_cap, gate_elems))) return rc;

    // rope + append of rows [i0, i0 + n): causality is enforced by the mask, not by write order
    auto append_rows = [&](int i0, int n) -> int {
        const int max_items = 65535;
        for (int j0 = i0; j0 < i0 + n; j0 += max_items) {
            const int cnt = std::min(max_items, i0 + n - j0);
            Items it{};
            it.mode = 1;
            it.seq0 = seq;
            it.base_pos = base_pos + j0;
            it.n = cnt;
            const void* fq = dq + (size_t)j0 * c->q_dim * es;
            const void* fk = dk + (size_t)j0 * c->kv_dim * es;
            const void* fv = dv + (size_t)j0 * c->kv_dim * es;
            int in_bf16 = in_dtype == GGR_DTYPE_BF16;
            int r = apply_fixups(c, layer, cnt, &fq, &fk, &fv, &in_bf16);
            if (r) return r;
            r = launch_rope_append(c, layer, it, RF_ROTATE | RF_WRITE_Q | RF_APPEND, in_bf16, fq, fk, fv,
                                   tc ? nullptr : c->d_qrot + (size_t)j0 * c->q_dim,
                                   tc ? c->d_qrot_h + (size_t)j0 * c->q_dim : nullptr, nullptr);
            if (r) return r;
        }
        return GGR_OK;
    };
    // attention of rows [i0, i0 + n) over the cache (their own rows must already be appended)
    auto attend_rows = [&](int i0, int n) -> int {
        if (tc) {
            PrefillTcArgs a{};
            a.kv = c->kv;
            a.vis = visibility(c, layer);
            a.layer = layer;
            a.seq = seq;
            a.base_pos = base_pos + i0;
            a.m = n;
            a.q = c->d_qrot_h + (size_t)i0 * c->q_dim;
            a.out = dout + (size_t)i0 * c->q_dim;
            a.score_scale = (c->cfg.scale_mode == GGR_SCALE_SCORE ? c->attn_scale : 1.0f) * kLog2e;
            a.err = c->d_err;
            a.sched = c->d_sched;
            // the rope / append kernel of these rows is the launch right in front of this one (event records of the
            // per-kernel timing would come between them)
            a.dependent = c->timing ? 0 : 1;
            if (gate) {
                a.gate = dgate + (size_t)i0 * gate_row * es;
                a.gate_bf16 = in_dtype == GGR_DTYPE_BF16;
                a.gate_head_stride = gate_head_stride;
            }
#ifdef GGR_TC_TRACE
            a.trace = g_tc_trace;
#endif
            std::string msg;
            int r;
            {
                LaunchTimer t(c, 0);
                r = wide ? launch_prefill_tc_wide(a, c->tmK64, c->tmV64, c->cfg.device, c->stream, &msg)
                         : launch_prefill_tc(a, c->tmK, c->tmV, c->cfg.device, c->sm_count, c->stream, &msg);
            }
            if (r) return fail(c, r, msg);
            c->launches++;
            return GGR_OK;
        }
        const int max_items = 65535;
        for (int j0 = i0; j0 < i0 + n; j0 += max_items) {
            const int cnt = std::min(max_items, i0 + n - j0);
            Items it{};
            it.mode = 1;
            it.seq0 = seq;
            it.base_pos = base_pos + j0;
            it.n = cnt;
            // widest visible range of the rows (ranges end at pos + 1 or at a block end)
            int vs, ve;
            visible_host(c, layer, base_pos + j0 + cnt - 1, &vs, &ve);
            int t_max = std::max(1, ve - vs);
            visible_host(c, layer, base_pos + j0, &vs, &ve);
            t_max = std::max(t_max, ve - vs);
            GateSpec gs{nullptr, gate_head_stride, 0};
            if (gate) {
                if (widen_gate) {
                    const size_t off = (size_t)j0 * gate_row, cnt_e = ((size_t)cnt * c->kv.Hq - 1) * gate_head_stride + c->D;
                    gate_to_f32_kernel<<<(unsigned)std::min<size_t>(1024, (cnt_e + 255) / 256), 256, 0, c->stream>>>(
                        reinterpret_cast<const __nv_bfloat16*>(dgate) + off, c->d_gate_f32 + off, cnt_e);
                    CUDA_TRY(c, cudaGetLastError());
                    c->launches++;
                    gs.p = c->d_gate_f32 + off;
                } else {
                    gs.p = reinterpret_cast<const float*>(dgate) + (size_t)j0 * gate_row;
                }
            }
            int r = launch_attention(c, layer, it, t_max, c->d_qrot + (size_t)j0 * c->q_dim, dout + (size_t)j0 * c->q_dim,
                                     nullptr, false, nullptr, nullptr, &gs);
            if (r) return r;
        }
        return GGR_OK;
    };

    if (!host) {
        if ((rc = append_rows(0, m))) return rc;
        return attend_rows(0, m);
    }

    // Host buffers: rows move in pieces so that the copy-in of piece p+1, the kernels of piece p and the
    // copy-out of piece p-1 overlap (three streams). A staged image block needs all its rows appended
    // before any row attends, so it is one piece.
    std::vector<std::pair<int, int>> pieces;  // (first row, rows)
    if (block_mode) {
        pieces.push_back({0, m});
    } else {
        // a smaller first piece: nothing overlaps its copy-in, so the output stream starts that much earlier
        // (32-layer S=4096 pass: 57.9 ms with 1024 rows first, 56.2 ms with 512 or 256, 57.2 ms with 128)
        const int first_rows = 512;
        int i0 = 0;
        while (i0 < m) {
            const int n = std::min(i0 == 0 ? first_rows : 1024, m - i0);
            pieces.push_back({i0, n});
            i0 += n;
        }
    }
    const int n_pieces = (int)pieces.size();
    if ((rc = ensure_copy_streams(c, n_pieces))) return rc;
    for (int p = 0; p < n_pieces; ++p) {
        const int i0 = pieces[p].first, n = pieces[p].second;
        const size_t qo = (size_t)i0 * c->q_dim * es, ko = (size_t)i0 * c->kv_dim * es;
        CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[0] + qo, static_cast<const unsigned char*>(q) + qo, (size_t)n * c->q_dim * es,
                                    cudaMemcpyHostToDevice, c->copy_in));
        CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[1] + ko, static_cast<const unsigned char*>(k) + ko, (size_t)n * c->kv_dim * es,
                                    cudaMemcpyHostToDevice, c->copy_in));
        CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[2] + ko, static_cast<const unsigned char*>(v) + ko, (size_t)n * c->kv_dim * es,
                                    cudaMemcpyHostToDevice, c->copy_in));
        if (gate) {
            const size_t go = (size_t)i0 * gate_row * es;
            const size_t gn = (((size_t)n * c->kv.Hq - 1) * gate_head_stride + c->D) * es;
            CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[4] + go, static_cast<const unsigned char*>(gate) + go, gn,
                                        cudaMemcpyHostToDevice, c->copy_in));
        }
        CUDA_TRY(c, cudaEventRecord(c->ev_in[p], c->copy_in));
        CUDA_TRY(c, cudaStreamWaitEvent(c->stream, c->ev_in[p], 0));
        if ((rc = append_rows(i0, n)) || (rc = attend_rows(i0, n))) {
            // copies of this and earlier pieces may still be in flight on buffers the next call may free
            cudaStreamSynchronize(c->copy_in);
            cudaStreamSynchronize(c->copy_out);
            cudaStreamSynchronize(c->stream);
            return rc;
        }
        CUDA_TRY(c, cudaEventRecord(c->ev_done[p], c->stream));
        CUDA_TRY(c, cudaStreamWaitEvent(c->copy_out, c->ev_done[p], 0));
        CUDA_TRY(c, cudaMemcpyAsync(out + (size_t)i0 * c->q_dim, dout + (size_t)i0 * c->q_dim,
                                    (size_t)n * c->q_dim * sizeof(float), cudaMemcpyDeviceToHost, c->copy_out));
    }
    CUDA_TRY(c, cudaStreamSynchronize(c->copy_out));
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    if (c->h_err && *c->h_err) {
        *c->h_err = 0;
        return fail(c, GGR_ERR_TIMEOUT, "a bounded wait inside the prefill kernel ran out");
    }
    return GGR_OK;
}

}  // namespace

extern "C" {

int ggr_attn_abi_version(void) { return GGR_ATTN_ABI_VERSION; }

void ggr_attn_config_init(ggr_attn_config* cfg) {
    if (!cfg) return;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->struct_size = (int32_t)sizeof(*cfg);
    cfg->max_batch = 1;
    cfg->rope_theta = 500000.0f;    // src/vendors/llama.rs:13-15
    cfg->rope_theta_swa = 10000.0f; // src/vendors/mod.rs:962
    cfg->rope_scale_global = 1.0f;
    cfg->rope_scale_local = 1.0f;
    cfg->swa_pattern = 6;           // src/vendors/mod.rs:963
    cfg->kv_format = GGR_KV_Q8_ROW;
    cfg->n_ranks = 1;
}

const char* ggr_attn_create_error(void) { return g_create_err.c_str(); }

int ggr_attn_create(const ggr_attn_config* cfg, ggr_attn_ctx** out) {
    auto bad = [&](int st, const char* msg) {
        g_create_err = msg;
        return st;
    };
    if (!cfg || !out) return bad(GGR_ERR_INVALID, "null argument");
    *out = nullptr;
    if (cfg->struct_size != (int32_t)sizeof(ggr_attn_config)) return bad(GGR_ERR_INVALID, "ggr_attn_config size mismatch");
    // src/engine/runtime/inference.rs:1533-1546
    for (float s : {cfg->rope_scale_global, cfg->rope_scale_local})
        if (!std::isfinite(s) || s <= 0.0f) return bad(GGR_ERR_INVALID, "RoPE frequency scales must be finite and positive");
    if (cfg->n_layer_windows != 0) {
        bool wrong = cfg->n_layer_windows != cfg->n_layers || !cfg->layer_windows;
        for (int i = 0; !wrong && i < cfg->n_layer_windows; ++i) wrong = cfg->layer_windows[i] < 0;
        if (wrong) return bad(GGR_ERR_INVALID, "attention policy requires one positive window or global entry per layer");
    }
    if (cfg->n_layers <= 0 || cfg->n_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->head_dim <= 0 || cfg->seq_len <= 0 ||
        cfg->max_batch <= 0 || cfg->n_heads % cfg->n_kv_heads != 0)
        return bad(GGR_ERR_INVALID, "invalid attention shape");
    if (cfg->head_dim % 8 != 0 || cfg->head_dim > 256)
        return bad(GGR_ERR_UNSUPPORTED, "head_dim must be a multiple of 8 and at most 256");
    if (cfg->kv_format < GGR_KV_F32 || cfg->kv_format > GGR_KV_TURBO) return bad(GGR_ERR_INVALID, "unknown kv_format");
    if (cfg->kv_format == GGR_KV_TURBO && cfg->head_dim != 64 && cfg->head_dim != 128 && cfg->head_dim != 256)
        return bad(GGR_ERR_UNSUPPORTED, "the TurboQuant cache is built for head_dim 64, 128 or 256");
    if (cfg->kv_format == GGR_KV_Q8_BLOCK32 && cfg->head_dim % 32 != 0)
        return bad(GGR_ERR_UNSUPPORTED, "q8 block scales need head_dim to be a multiple of 32");
    int rope_dim = cfg->rope_dim > 0 ? cfg->rope_dim : cfg->head_dim;
    if (rope_dim > cfg->head_dim || (rope_dim & 1)) return bad(GGR_ERR_INVALID, "rope_dim must be even and at most head_dim");
    if (cfg->rope_style == GGR_ROPE_ADJACENT && rope_dim != cfg->head_dim)
        return bad(GGR_ERR_INVALID, "adjacent-pair RoPE rotates the whole head: rope_dim must equal head_dim");
    if (!(cfg->rope_theta > 0.0f) || !std::isfinite(cfg->rope_theta)) return bad(GGR_ERR_INVALID, "rope_theta must be positive");
    int shard_begin = 0, shard_count = cfg->seq_len;
    if (cfg->shard_mode == GGR_SHARD_KV_SEQUENCE) {
        shard_begin = cfg->shard_pos_begin;
        shard_count = cfg->shard_pos_count;
        if (shard_begin < 0 || shard_count <= 0 || (int64_t)shard_begin + shard_count > cfg->seq_len)
            return bad(GGR_ERR_INVALID, "shard position range outside the cache");
    } else if (cfg->shard_mode != GGR_SHARD_NONE) {
        return bad(GGR_ERR_INVALID, "unknown shard_mode");
    }

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) return bad(GGR_ERR_CUDA, "no CUDA device is available");
    if (cfg->device < 0 || cfg->device >= ndev) return bad(GGR_ERR_INVALID, "device ordinal out of range");
    DeviceGuard guard(cfg->device);

    ggr_attn_ctx* c = new ggr_attn_ctx();
    c->cfg = *cfg;
    c->cfg.layer_windows = nullptr;
    if (cfg->n_layer_windows) c->windows.assign(cfg->layer_windows, cfg->layer_windows + cfg->n_layer_windows);
    c->D = cfg->head_dim;
    c->kv_dim = cfg->n_kv_heads * c->D;
    c->q_dim = cfg->n_heads * c->D;
    c->G = cfg->n_heads / cfg->n_kv_heads;
    c->rope_dim = rope_dim;
    c->rope_half = rope_dim / 2;
    c->attn_scale = 1.0f / sqrtf((float)c->D);  // src/engine/runtime/inference.rs:1745
    c->shard_begin = shard_begin;
    c->shard_count = shard_count;

    auto cleanup = [&](int st, const std::string& msg) {
        g_create_err = msg;
        ggr_attn_destroy(c);
        return st;
    };
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess) return cleanup(GGR_ERR_CUDA, "cudaGetDeviceProperties failed");
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return cleanup(GGR_ERR_CUDA, "cudaStreamCreate failed");
    c->stream = c->own_stream;

    // RoPE frequency tables (src/engine/runtime/inference.rs:1590-1609), computed on the host like the reference
    std::vector<float> fr(c->rope_half), frs(c->rope_half);
    const float swa_theta = cfg->rope_theta_swa > 0.0f ? cfg->rope_theta_swa : 10000.0f;
    for (int i = 0; i < c->rope_half; ++i) {
        const float e = (float)(i * 2) / (float)rope_dim;
        fr[i] = 1.0f / powf(cfg->rope_theta, e);
        frs[i] = 1.0f / powf(swa_theta, e);
    }
    const size_t fb = std::max<size_t>(1, c->rope_half) * sizeof(float);
    if (cudaMalloc((void**)&c->d_freqs, fb) != cudaSuccess || cudaMalloc((void**)&c->d_freqs_swa, fb) != cudaSuccess)
        return cleanup(GGR_ERR_ALLOC, "unable to allocate RoPE tables");
    cudaMemcpy(c->d_freqs, fr.data(), c->rope_half * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemcpy(c->d_freqs_swa, frs.data(), c->rope_half * sizeof(float), cudaMemcpyHostToDevice);

    // KV cache (src/engine/runtime/inference.rs:1615-1630)
    KvView& kv = c->kv;
    kv.fmt = cfg->kv_format;
    kv.D = c->D;
    kv.kv_dim = c->kv_dim;
    kv.Hkv = cfg->n_kv_heads;
    kv.Hq = cfg->n_heads;
    kv.G = c->G;
    kv.n_layers = cfg->n_layers;
    kv.rows = shard_count;
    kv.pos_begin = shard_begin;
    kv.elem_bytes = elem_bytes_of(cfg->kv_format);
    kv.n_scales = cfg->kv_format == GGR_KV_Q8_ROW ? 1 : (cfg->kv_format == GGR_KV_Q8_BLOCK32 ? c->kv_dim / 32 : 0);
    const bool turbo = cfg->kv_format == GGR_KV_TURBO;
    if (turbo) kv.n_scales = cfg->n_kv_heads;  // sigma per (row, kv head): src/engine/runtime/inference.rs:1717
    const size_t rows = (size_t)cfg->max_batch * cfg->n_layers * shard_count;
    // TurboQuant: 2 bits per element in k / v, 1 bit per element in k_sign / v_sign (:1658-1662)
    const size_t bytes = turbo ? (rows * c->kv_dim + 3) / 4 : rows * c->kv_dim * kv.elem_bytes;
    char buf[160];
    if (cudaMalloc(&kv.k, bytes) != cudaSuccess || cudaMalloc(&kv.v, bytes) != cudaSuccess) {
        cudaGetLastError();
        // wording follows src/engine/runtime/inference.rs:130-164
        snprintf(buf, sizeof buf, "unable to allocate kv cache (%zu bytes). Try reducing the context size.", 2 * bytes);
        return cleanup(GGR_ERR_ALLOC, buf);
    }
    cudaMemsetAsync(kv.k, 0, bytes, c->stream);
    cudaMemsetAsync(kv.v, 0, bytes, c->stream);
    if (kv.n_scales) {
        const size_t sb = rows * kv.n_scales * sizeof(float);
        if (cudaMalloc((void**)&kv.ks, sb) != cudaSuccess || cudaMalloc((void**)&kv.vs, sb) != cudaSuccess) {
            cudaGetLastError();
            return cleanup(GGR_ERR_ALLOC, "unable to allocate kv scale buffers");
        }
        cudaMemsetAsync(kv.ks, 0, sb, c->stream);
        cudaMemsetAsync(kv.vs, 0, sb, c->stream);
    }
    if (turbo) {
        const size_t sign_bytes = (rows * c->kv_dim + 7) / 8, aux = rows * cfg->n_kv_heads * sizeof(float);
        if (cudaMalloc((void**)&kv.k_sign, sign_bytes) != cudaSuccess || cudaMalloc((void**)&kv.v_sign, sign_bytes) != cudaSuccess ||
            cudaMalloc((void**)&kv.k_rn, aux) != cudaSuccess || cudaMalloc((void**)&kv.v_rn, aux) != cudaSuccess) {
            cudaGetLastError();
            return cleanup(GGR_ERR_ALLOC, "unable to allocate the TurboQuant sign and norm buffers");
        }
        cudaMemsetAsync(kv.k_sign, 0, sign_bytes, c->stream);
        cudaMemsetAsync(kv.v_sign, 0, sign_bytes, c->stream);
        cudaMemsetAsync(kv.k_rn, 0, aux, c->stream);
        cudaMemsetAsync(kv.v_rn, 0, aux, c->stream);
        // sign tables of the four transforms (:370-395): bit 1 = negate, [slot][layer][kv_head][D / 8]
        const std::vector<unsigned char> table = ggr_turbo_sign_table(cfg->n_layers, cfg->n_kv_heads, c->D);
        if (cudaMalloc((void**)&c->d_turbo_signs, table.size()) != cudaSuccess) {
            cudaGetLastError();
            return cleanup(GGR_ERR_ALLOC, "unable to allocate the TurboQuant sign tables");
        }
        if (cudaMemcpyAsync(c->d_turbo_signs, table.data(), table.size(), cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
            cudaStreamSynchronize(c->stream) != cudaSuccess)
            return cleanup(GGR_ERR_CUDA, "unable to upload the TurboQuant sign tables");
        kv.turbo_signs = c->d_turbo_signs;
    }
    if (cudaHostAlloc((void**)&c->h_err, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&c->d_err, c->h_err, 0) != cudaSuccess) {
        cudaGetLastError();
        return cleanup(GGR_ERR_ALLOC, "unable to allocate the error word");
    }
    *c->h_err = 0;
    if (cudaMalloc((void**)&c->d_sched, 2 * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return cleanup(GGR_ERR_ALLOC, "unable to allocate the prefill work counters");
    }
    cudaMemsetAsync(c->d_sched, 0, 2 * sizeof(int), c->stream);
    if (prefill_tc_shape_ok(kv.fmt, c->D) && rows < ((size_t)1 << 31)) {
        c->have_tmaps = make_tmap_bf16(&c->tmK, kv.k, (uint64_t)c->kv_dim, (uint64_t)rows) &&
                        make_tmap_bf16(&c->tmV, kv.v, (uint64_t)c->kv_dim, (uint64_t)rows);
    }
    if (kv.fmt == KV_BF16 && c->D == 256 && rows < ((size_t)1 << 31)) {
        c->have_tmaps64 = make_tmap_bf16(&c->tmK64, kv.k, (uint64_t)c->kv_dim, (uint64_t)rows, kTwBN) &&
                          make_tmap_bf16(&c->tmV64, kv.v, (uint64_t)c->kv_dim, (uint64_t)rows, kTwBN);
    }
    if (kv.fmt == KV_BF16 && mma_tma_decode_supported(c->D) && rows < ((size_t)1 << 31)) {
        c->have_tmaps16 = make_tmap_bf16(&c->tmK16, kv.k, (uint64_t)c->kv_dim, (uint64_t)rows, kTmaTK) &&
                          make_tmap_bf16(&c->tmV16, kv.v, (uint64_t)c->kv_dim, (uint64_t)rows, kTmaTK);
    }
    if (cfg->exchange_wait_us < 0) return cleanup(GGR_ERR_INVALID, "exchange_wait_us must not be negative");
    c->x_wait_ns = cfg->exchange_wait_us > 0 ? (unsigned long long)cfg->exchange_wait_us * 1000ull : 1000000000ull;
    // decode scratch for max_batch sequences, so that the token loop never allocates (see ggr_attn_reserve)
    if (int rr = reserve_decode(c, std::min(cfg->max_batch, kMaxArgItems))) return cleanup(rr, c->err);
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) return cleanup(GGR_ERR_CUDA, "device initialisation failed");
    g_create_err.clear();
    *out = c;
    return GGR_OK;
}

void ggr_attn_destroy(ggr_attn_ctx* c) {
    if (!c) return;
    DeviceGuard guard(c->cfg.device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    cudaFree(c->kv.k);
    cudaFree(c->kv.v);
    cudaFree(c->kv.ks);
    cudaFree(c->kv.vs);
    cudaFree(c->kv.k_sign);
    cudaFree(c->kv.v_sign);
    cudaFree(c->kv.k_rn);
    cudaFree(c->kv.v_rn);
    cudaFree(c->d_turbo_signs);
    cudaFree(c->d_krot);
    cudaFree(c->d_freqs);
    cudaFree(c->d_freqs_swa);
    cudaFree(c->d_plan);
    cudaFree(c->d_blocks);
    cudaFree(c->d_qrot);
    cudaFree(c->d_qrot_h);
    cudaFree(c->d_part);
    cudaFree(c->d_counters);
    for (auto* p : c->d_stage) cudaFree(p);
    cudaFree(c->d_gate_f32);
    cudaFree(c->d_px);
    cudaFree(c->d_pqkv);
    cudaFree(c->d_patt);
    cudaFree(c->d_pout);
    cudaFree(c->d_pact);
    cudaFree(c->d_pqkv_h);
    cudaFree(c->d_pin_in);
    if (c->h_pin) cudaFreeHost(c->h_pin);
    for (int r = 0; r < kMaxPeers; ++r)
        if (c->x_opened[r]) cudaIpcCloseMemHandle(c->x_peer[r]);
    cudaFree(c->x_local);
    cudaFree(c->d_done);
    for (auto* p : c->d_fix) cudaFree(p);
    for (auto& f : c->fixups)
        for (float* p : {f.q_bias, f.k_bias, f.v_bias, f.q_norm, f.k_norm}) cudaFree(p);
    if (c->h_err) cudaFreeHost(c->h_err);
    if (c->d_sched) cudaFree(c->d_sched);
    for (auto e : c->ev_in) cudaEventDestroy(e);
    for (auto e : c->ev_done) cudaEventDestroy(e);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    for (auto& pool : c->ev)
        for (auto& pr : pool) {
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
}

const char* ggr_attn_last_error(const ggr_attn_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }
int64_t ggr_attn_launch_count(const ggr_attn_ctx* ctx) { return ctx ? ctx->launches : 0; }
int32_t ggr_attn_last_split_count(const ggr_attn_ctx* ctx) { return ctx ? ctx->last_splits : 0; }

int ggr_attn_set_stream(ggr_attn_ctx* c, void* cuda_stream) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    c->stream = cuda_stream ? (cudaStream_t)cuda_stream : c->own_stream;
    return GGR_OK;
}

int ggr_attn_synchronize(ggr_attn_ctx* c) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return take_device_error(c, "a bounded wait inside a kernel ran out");
}

int ggr_attn_set_kernel_timing(ggr_attn_ctx* c, int32_t enable) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    c->timing = enable != 0;
    for (auto& u : c->ev_used) u = 0;
    return GGR_OK;
}

int ggr_attn_kernel_time(ggr_attn_ctx* c, int32_t kind, double* total_ms, int64_t* launches, int32_t reset) {
    if (!c || kind < 0 || kind > 3 || !total_ms || !launches) return fail(c, GGR_ERR_INVALID, "invalid timing query");
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    double sum = 0.0;
    for (size_t i = 0; i < c->ev_used[kind]; ++i) {
        float ms = 0.f;
        CUDA_TRY(c, cudaEventElapsedTime(&ms, c->ev[kind][i].first, c->ev[kind][i].second));
        sum += ms;
    }
    *total_ms = sum;
    *launches = (int64_t)c->ev_used[kind];
    if (reset) c->ev_used[kind] = 0;
    return GGR_OK;
}

int ggr_attn_kv_device_ptrs(ggr_attn_ctx* c, void** k, void** v, float** k_scale, float** v_scale,
                            uint64_t* array_bytes) {
    if (!c) return GGR_ERR_INVALID;
    if (k) *k = c->kv.k;
    if (v) *v = c->kv.v;
    if (k_scale) *k_scale = c->kv.ks;
    if (v_scale) *v_scale = c->kv.vs;
    if (array_bytes) {
        const uint64_t elems = (uint64_t)c->cfg.max_batch * c->cfg.n_layers * c->shard_count * c->kv_dim;
        *array_bytes = c->kv.fmt == KV_TURBO ? (elems + 3) / 4 : elems * c->kv.elem_bytes;  // TurboQuant: the code arrays
    }
    return GGR_OK;
}

int ggr_attn_set_position_plan(ggr_attn_ctx* c, const int32_t* thw, int32_t n, int32_t next_text_pos) {
    if (!c || n < 0 || (n > 0 && !thw) || next_text_pos < 0) return fail(c, GGR_ERR_INVALID, "invalid position plan");
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    cudaFree(c->d_plan);
    c->d_plan = nullptr;
    c->plan_len = n;
    c->next_text = next_text_pos;
    c->has_plan = (n > 0 || next_text_pos != 0) ? 1 : 0;
    if (n > 0) {
        if (cudaMalloc((void**)&c->d_plan, (size_t)n * 3 * sizeof(int)) != cudaSuccess)
            return fail(c, GGR_ERR_ALLOC, "unable to allocate the position plan");
        CUDA_TRY(c, cudaMemcpy(c->d_plan, thw, (size_t)n * 3 * sizeof(int), cudaMemcpyHostToDevice));
    }
    return GGR_OK;
}

int ggr_attn_set_media_blocks(ggr_attn_ctx* c, const int32_t* start_len, int32_t n, int32_t prompt_tokens) {
    if (!c || n < 0 || (n > 0 && !start_len)) return fail(c, GGR_ERR_INVALID, "invalid media blocks");
    std::vector<int64_t> sl(2 * (size_t)n);
    for (int i = 0; i < 2 * n; ++i) sl[i] = start_len[i];
    if (ggr_media_plan_validate(sl.data(), n, prompt_tokens) != GGR_OK)
        return fail(c, GGR_ERR_INVALID,
                    "image attention blocks must be nonempty, ordered, disjoint, and within the prompt");
    DeviceGuard guard(c->cfg.device);
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    cudaFree(c->d_blocks);
    c->d_blocks = nullptr;
    c->blocks.clear();
    for (int i = 0; i < n; ++i) c->blocks.push_back(make_int2(start_len[2 * i], start_len[2 * i + 1]));
    if (n > 0) {
        if (cudaMalloc((void**)&c->d_blocks, (size_t)n * sizeof(int2)) != cudaSuccess)
            return fail(c, GGR_ERR_ALLOC, "unable to allocate media blocks");
        CUDA_TRY(c, cudaMemcpy(c->d_blocks, c->blocks.data(), (size_t)n * sizeof(int2), cudaMemcpyHostToDevice));
    }
    return GGR_OK;
}

int ggr_attn_visible_keys(const ggr_attn_ctx* c, int32_t layer, int32_t pos, int32_t* start, int32_t* end) {
    if (!c || !start || !end || layer < 0 || layer >= c->cfg.n_layers || pos < 0) return GGR_ERR_INVALID;
    visible_host(c, layer, pos, start, end);
    return GGR_OK;
}

int ggr_attn_decode(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* q, const float* k,
                    const float* v, float* out, int32_t ptr_kind) {
    if (!out) return fail(c, GGR_ERR_INVALID, "null buffer");
    return decode_common(c, layer, pos, B, q, k, v, out, nullptr, ptr_kind);
}

int ggr_attn_decode_gated(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* q, const float* k,
                          const float* v, const float* gate, int32_t gate_head_stride, float* out, int32_t ptr_kind) {
    if (!out || !gate) return fail(c, GGR_ERR_INVALID, "null buffer");
    return decode_common(c, layer, pos, B, q, k, v, out, nullptr, ptr_kind, gate, gate_head_stride);
}

int ggr_attn_reserve(ggr_attn_ctx* c, int32_t B) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (B <= 0 || B > c->cfg.max_batch) return fail(c, GGR_ERR_RANGE, "batch larger than max_batch");
    return reserve_decode(c, B);
}

int ggr_attn_decode_partial(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                            const float* k, const float* v, float* partial, int32_t ptr_kind) {
    if (!partial) return fail(c, GGR_ERR_INVALID, "null buffer");
    return decode_common(c, layer, pos, B, q, k, v, nullptr, partial, ptr_kind);
}

int ggr_attn_combine_partials(ggr_attn_ctx* c, const float* parts, int32_t n_parts, int32_t B, float* out,
                              int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    if (!parts || !out || n_parts <= 0 || B <= 0) return fail(c, GGR_ERR_INVALID, "invalid combine arguments");
    DeviceGuard guard(c->cfg.device);
    const size_t in_bytes = (size_t)n_parts * B * c->kv.Hq * (c->D + 2) * sizeof(float);
    const size_t out_bytes = (size_t)B * c->q_dim * sizeof(float);
    const void* dp;
    int rc = stage_in(c, 0, parts, in_bytes, ptr_kind, &dp);
    if (rc) return rc;
    float* dout = out;
    if (ptr_kind == GGR_PTR_HOST) {
        if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], out_bytes))) return rc;
        dout = reinterpret_cast<float*>(c->d_stage[3]);
    }
    {
        LaunchTimer t(c, 2);
        combine_partials_kernel<<<dim3(c->kv.Hq, B), 128, 0, c->stream>>>(reinterpret_cast<const float*>(dp), n_parts,
                                                                          B, c->kv.Hq, c->D, dout, nullptr, 0);
    }
    CUDA_TRY(c, cudaGetLastError());
    c->launches++;
    if (ptr_kind == GGR_PTR_HOST) {
        CUDA_TRY(c, cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    }
    return GGR_OK;
}

int ggr_attn_prefill(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const void* q,
                     const void* k, const void* v, int32_t in_dtype, float* out, int32_t ptr_kind) {
    return prefill_common(c, layer, seq, base_pos, m, q, k, v, in_dtype, out, ptr_kind, false);
}

int ggr_attn_prefill_gated(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const void* q,
                           const void* k, const void* v, const void* gate, int32_t gate_head_stride, int32_t in_dtype,
                           float* out, int32_t ptr_kind) {
    if (!gate) return fail(c, GGR_ERR_INVALID, "null buffer");
    return prefill_common(c, layer, seq, base_pos, m, q, k, v, in_dtype, out, ptr_kind, false, gate, gate_head_stride);
}

int ggr_attn_prefill_block(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const void* q,
                           const void* k, const void* v, int32_t in_dtype, float* out, int32_t ptr_kind) {
    return prefill_common(c, layer, seq, base_pos, m, q, k, v, in_dtype, out, ptr_kind, true);
}

int ggr_attn_apply_rope_qk(ggr_attn_ctx* c, int32_t layer, int32_t pos, float* q, float* k, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!q || !k || pos < 0) return fail(c, GGR_ERR_INVALID, "invalid rope arguments");
    const size_t qb = (size_t)c->q_dim * sizeof(float), kb = (size_t)c->kv_dim * sizeof(float);
    // the rotation reads pairs, so it never runs in place: inputs go through staging
    if ((rc = ensure(c, &c->d_stage[0], &c->stage_cap[0], qb))) return rc;
    if ((rc = ensure(c, &c->d_stage[1], &c->stage_cap[1], kb))) return rc;
    if ((rc = ensure(c, &c->d_stage[2], &c->stage_cap[2], kb))) return rc;
    if ((rc = ensure(c, &c->d_qrot, &c->qrot_cap, (size_t)c->q_dim))) return rc;
    const cudaMemcpyKind in_kind = ptr_kind == GGR_PTR_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const cudaMemcpyKind out_kind = ptr_kind == GGR_PTR_HOST ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[0], q, qb, in_kind, c->stream));
    CUDA_TRY(c, cudaMemcpyAsync(c->d_stage[1], k, kb, in_kind, c->stream));
    Items it{};
    it.mode = 0;
    it.seq0 = 0;
    it.n = 1;
    it.pos[0] = pos;
    rc = launch_rope_append(c, layer, it, RF_ROTATE | RF_WRITE_Q | RF_WRITE_K, 0, c->d_stage[0], c->d_stage[1], nullptr,
                            c->d_qrot, nullptr, reinterpret_cast<float*>(c->d_stage[2]));
    if (rc) return rc;
    CUDA_TRY(c, cudaMemcpyAsync(q, c->d_qrot, qb, out_kind, c->stream));
    CUDA_TRY(c, cudaMemcpyAsync(k, c->d_stage[2], kb, out_kind, c->stream));
    if (ptr_kind == GGR_PTR_HOST) CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return GGR_OK;
}

int ggr_attn_kv_write_token(ggr_attn_ctx* c, int32_t seq, int32_t layer, int32_t pos, const float* k, const float* v,
                            int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!k || !v) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (seq < 0 || seq >= c->cfg.max_batch || pos < 0 || pos >= c->cfg.seq_len)
        return fail(c, GGR_ERR_RANGE, "cache row outside the cache");
    const size_t kb = (size_t)c->kv_dim * sizeof(float);
    const void *dk, *dv;
    if ((rc = stage_in(c, 1, k, kb, ptr_kind, &dk))) return rc;
    if ((rc = stage_in(c, 2, v, kb, ptr_kind, &dv))) return rc;
    Items it{};
    it.mode = 0;
    it.seq0 = seq;
    it.n = 1;
    it.pos[0] = pos;
    rc = launch_rope_append(c, layer, it, RF_APPEND, 0, nullptr, dk, dv, nullptr, nullptr, nullptr);
    if (rc) return rc;
    if (ptr_kind == GGR_PTR_HOST) CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return GGR_OK;
}

int ggr_attn_attention_token(ggr_attn_ctx* c, int32_t seq, int32_t layer, int32_t pos, const float* q, float* out,
                             int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!q || !out) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (seq < 0 || seq >= c->cfg.max_batch || pos < 0 || pos >= c->cfg.seq_len)
        return fail(c, GGR_ERR_RANGE, "cache row outside the cache");
    if (c->cfg.shard_mode != GGR_SHARD_NONE) return fail(c, GGR_ERR_UNSUPPORTED, "use ggr_attn_decode_partial on a shard");
    const size_t qb = (size_t)c->q_dim * sizeof(float);
    const void* dq;
    if ((rc = stage_in(c, 0, q, qb, ptr_kind, &dq))) return rc;
    float* dout = out;
    if (ptr_kind == GGR_PTR_HOST) {
        if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], qb))) return rc;
        dout = reinterpret_cast<float*>(c->d_stage[3]);
    }
    Items it{};
    it.mode = 0;
    it.seq0 = seq;
    it.n = 1;
    it.pos[0] = pos;
    const int t_max = t_max_of(c, layer, &pos, 1);
    rc = launch_attention(c, layer, it, t_max, reinterpret_cast<const float*>(dq), dout, nullptr, true);
    if (rc) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        CUDA_TRY(c, cudaMemcpyAsync(out, dout, qb, cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    }
    return GGR_OK;
}

static int kv_rows_check(ggr_attn_ctx* c, int layer, int seq, int row0, int nrows) {
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (seq < 0 || seq >= c->cfg.max_batch || row0 < c->shard_begin || nrows < 0 ||
        (int64_t)row0 + nrows > (int64_t)c->shard_begin + c->shard_count)
        return fail(c, GGR_ERR_RANGE, "rows outside the cache");
    return GGR_OK;
}

// One row range of one layer as contiguous spans: {device base, bytes per row} pairs of every array the format keeps.
struct RowSpans {
    int n;
    unsigned char* dev[8];
    size_t row_bytes[8];
};

static RowSpans row_spans(const ggr_attn_ctx* c) {
    RowSpans r{};
    const KvView& kv = c->kv;
    const size_t n = (size_t)c->kv_dim;
    if (kv.fmt == KV_TURBO) {
        const size_t h = (size_t)kv.Hkv * sizeof(float);
        unsigned char* dev[8] = {(unsigned char*)kv.k, (unsigned char*)kv.v, kv.k_sign, kv.v_sign, (unsigned char*)kv.ks,
                                 (unsigned char*)kv.vs, (unsigned char*)kv.k_rn, (unsigned char*)kv.v_rn};
        const size_t rb[8] = {n / 4, n / 4, n / 8, n / 8, h, h, h, h};
        r.n = 8;
        for (int i = 0; i < 8; ++i) r.dev[i] = dev[i], r.row_bytes[i] = rb[i];
    } else {
        const size_t sb = (size_t)kv.n_scales * sizeof(float);
        unsigned char* dev[4] = {(unsigned char*)kv.k, (unsigned char*)kv.v, (unsigned char*)kv.ks, (unsigned char*)kv.vs};
        const size_t rb[4] = {n, n, sb, sb};
        r.n = 4;
        for (int i = 0; i < 4; ++i) r.dev[i] = dev[i], r.row_bytes[i] = rb[i];
    }
    return r;
}

static int move_rows(ggr_attn_ctx* c, int layer, int seq, int row0, int nrows, void* const* host, bool to_host) {
    int rc = kv_rows_check(c, layer, seq, row0, nrows);
    if (rc) return rc;
    const RowSpans sp = row_spans(c);
    for (int i = 0; i < sp.n; ++i)
        if (!host[i]) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (nrows == 0) return GGR_OK;
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    const int64_t r = c->kv.row(seq, layer, row0);
    for (int i = 0; i < sp.n; ++i) {
        unsigned char* d = sp.dev[i] + (size_t)r * sp.row_bytes[i];
        const size_t nb = (size_t)nrows * sp.row_bytes[i];
        if (to_host)
            CUDA_TRY(c, cudaMemcpy(host[i], d, nb, cudaMemcpyDeviceToHost));
        else
            CUDA_TRY(c, cudaMemcpy(d, host[i], nb, cudaMemcpyHostToDevice));
    }
    return GGR_OK;
}

int ggr_attn_kv_export(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t row0, int32_t nrows, int8_t* k_q8,
                       int8_t* v_q8, float* k_scale, float* v_scale) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (c->kv.fmt != KV_Q8_ROW && c->kv.fmt != KV_Q8_BLOCK32)
        return fail(c, GGR_ERR_UNSUPPORTED, "export needs a q8 cache format (row or block-32 scales)");
    void* host[4] = {k_q8, v_q8, k_scale, v_scale};
    return move_rows(c, layer, seq, row0, nrows, host, true);
}

int ggr_attn_kv_import(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t row0, int32_t nrows, const int8_t* k_q8,
                       const int8_t* v_q8, const float* k_scale, const float* v_scale) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (c->kv.fmt != KV_Q8_ROW && c->kv.fmt != KV_Q8_BLOCK32)
        return fail(c, GGR_ERR_UNSUPPORTED, "import needs a q8 cache format (row or block-32 scales)");
    void* host[4] = {const_cast<int8_t*>(k_q8), const_cast<int8_t*>(v_q8), const_cast<float*>(k_scale),
                     const_cast<float*>(v_scale)};
    return move_rows(c, layer, seq, row0, nrows, host, false);
}

int ggr_attn_kv_export_turbo(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t row0, int32_t nrows, uint8_t* k_base,
                             uint8_t* v_base, uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale,
                             float* k_rnorm, float* v_rnorm) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (c->kv.fmt != KV_TURBO) return fail(c, GGR_ERR_UNSUPPORTED, "the cache is not in the TurboQuant format");
    void* host[8] = {k_base, v_base, k_sign, v_sign, k_scale, v_scale, k_rnorm, v_rnorm};
    return move_rows(c, layer, seq, row0, nrows, host, true);
}

int ggr_attn_kv_import_turbo(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t row0, int32_t nrows,
                             const uint8_t* k_base, const uint8_t* v_base, const uint8_t* k_sign, const uint8_t* v_sign,
                             const float* k_scale, const float* v_scale, const float* k_rnorm, const float* v_rnorm) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (c->kv.fmt != KV_TURBO) return fail(c, GGR_ERR_UNSUPPORTED, "the cache is not in the TurboQuant format");
    void* host[8] = {const_cast<uint8_t*>(k_base), const_cast<uint8_t*>(v_base), const_cast<uint8_t*>(k_sign),
                     const_cast<uint8_t*>(v_sign), const_cast<float*>(k_scale), const_cast<float*>(v_scale),
                     const_cast<float*>(k_rnorm), const_cast<float*>(v_rnorm)};
    return move_rows(c, layer, seq, row0, nrows, host, false);
}

int ggr_attn_kv_read_row(ggr_attn_ctx* c, int32_t seq, int32_t layer, int32_t pos, float* k_out, float* v_out) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = kv_rows_check(c, layer, seq, pos, 1);
    if (rc) return rc;
    if (c->kv.fmt == KV_TURBO)
        return fail(c, GGR_ERR_UNSUPPORTED, "a TurboQuant row has no element-wise decoding: read it with ggr_attn_kv_read_turbo");
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    const int64_t r = c->kv.row(seq, layer, pos);
    const int n = c->kv_dim, eb = c->kv.elem_bytes;
    std::vector<unsigned char> kb((size_t)n * eb), vb((size_t)n * eb);
    CUDA_TRY(c, cudaMemcpy(kb.data(), (unsigned char*)c->kv.k + r * n * eb, kb.size(), cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(vb.data(), (unsigned char*)c->kv.v + r * n * eb, vb.size(), cudaMemcpyDeviceToHost));
    std::vector<float> ks(std::max(1, c->kv.n_scales)), vs(std::max(1, c->kv.n_scales));
    if (c->kv.n_scales) {
        CUDA_TRY(c, cudaMemcpy(ks.data(), c->kv.ks + r * c->kv.n_scales, c->kv.n_scales * sizeof(float), cudaMemcpyDeviceToHost));
        CUDA_TRY(c, cudaMemcpy(vs.data(), c->kv.vs + r * c->kv.n_scales, c->kv.n_scales * sizeof(float), cudaMemcpyDeviceToHost));
    }
    for (int i = 0; i < n; ++i) {
        switch (c->kv.fmt) {
            case KV_F32:
                k_out[i] = reinterpret_cast<float*>(kb.data())[i];
                v_out[i] = reinterpret_cast<float*>(vb.data())[i];
                break;
            case KV_BF16: {
                uint32_t a = (uint32_t)reinterpret_cast<uint16_t*>(kb.data())[i] << 16;
                uint32_t b = (uint32_t)reinterpret_cast<uint16_t*>(vb.data())[i] << 16;
                std::memcpy(&k_out[i], &a, 4);
                std::memcpy(&v_out[i], &b, 4);
                break;
            }
            case KV_Q8_ROW:
                k_out[i] = (float)reinterpret_cast<int8_t*>(kb.data())[i] * ks[0];
                v_out[i] = (float)reinterpret_cast<int8_t*>(vb.data())[i] * vs[0];
                break;
            default:
                k_out[i] = (float)reinterpret_cast<int8_t*>(kb.data())[i] * ks[i / 32];
                v_out[i] = (float)reinterpret_cast<int8_t*>(vb.data())[i] * vs[i / 32];
                break;
        }
    }
    return GGR_OK;
}

int ggr_attn_kv_read_turbo(ggr_attn_ctx* c, int32_t seq, int32_t layer, int32_t pos, uint8_t* k_base, uint8_t* v_base,
                           uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale, float* k_rnorm,
                           float* v_rnorm) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = kv_rows_check(c, layer, seq, pos, 1);
    if (rc) return rc;
    if (c->kv.fmt != KV_TURBO) return fail(c, GGR_ERR_UNSUPPORTED, "the cache is not in the TurboQuant format");
    if (!k_base || !v_base || !k_sign || !v_sign || !k_scale || !v_scale || !k_rnorm || !v_rnorm)
        return fail(c, GGR_ERR_INVALID, "null buffer");
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    const int64_t r = c->kv.row(seq, layer, pos);
    const size_t n = (size_t)c->kv_dim, h = (size_t)c->kv.Hkv;
    CUDA_TRY(c, cudaMemcpy(k_base, (unsigned char*)c->kv.k + r * n / 4, n / 4, cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(v_base, (unsigned char*)c->kv.v + r * n / 4, n / 4, cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(k_sign, c->kv.k_sign + r * n / 8, n / 8, cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(v_sign, c->kv.v_sign + r * n / 8, n / 8, cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(k_scale, c->kv.ks + r * h, h * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(v_scale, c->kv.vs + r * h, h * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(k_rnorm, c->kv.k_rn + r * h, h * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_TRY(c, cudaMemcpy(v_rnorm, c->kv.v_rn + r * h, h * sizeof(float), cudaMemcpyDeviceToHost));
    return GGR_OK;
}

}  // extern "C"

// ---- allocation-free attention over the cache ----------------------------------------------------
//
// ggr_attn_attention_tokens_static is for hosts that must not allocate device memory while they
// decode: an engine that handed every byte of HBM to its KV caches and weights at start-up (so a
// cudaMalloc in the token loop could fail), or one that runs its decode step where an allocation's
// implicit device-wide synchronisation is not acceptable. The split-KV kernels need scratch (the
// per-split partial states and one ticket per (sequence, kv head)); here that scratch is a fixed
// array inside the library image instead of memory grown with cudaMalloc.

#define GGR_STATIC_SCRATCH_BYTES (8u << 20)
#define GGR_STATIC_TICKET_BYTES (64u << 10)
#define GGR_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char g_static_scratch[GGR_STATIC_SCRATCH_BYTES];

namespace {

std::mutex g_static_mu;
unsigned char* g_static_ptr[GGR_STATIC_MAX_DEVICES] = {};

// Device address of g_static_scratch on the context's device. In host code the array's name is
// only a handle, so the address comes from cudaGetSymbolAddress, asked once per device with that
// device current (the caller holds a DeviceGuard).
int static_scratch(ggr_attn_ctx* c, unsigned char** out) {
    const int dev = c->cfg.device;
    if (dev < 0 || dev >= GGR_STATIC_MAX_DEVICES) return fail(c, GGR_ERR_UNSUPPORTED, "device ordinal above 63");
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return fail(c, GGR_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
        g_static_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_static_ptr[dev];
    return GGR_OK;
}

}  // namespace

extern "C" int ggr_attn_attention_tokens_static(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B,
                                                const float* q_dev, float* out_dev) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!pos || !q_dev || !out_dev) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (c->cfg.shard_mode != GGR_SHARD_NONE) return fail(c, GGR_ERR_UNSUPPORTED, "not available on a KV-sequence shard");
    if (c->kv.fmt == KV_TURBO) return fail(c, GGR_ERR_UNSUPPORTED, "not available for the TurboQuant cache format");
    if (B <= 0 || B > c->cfg.max_batch) return fail(c, GGR_ERR_RANGE, "batch larger than max_batch");
    if (B > kMaxArgItems) return fail(c, GGR_ERR_RANGE, "the allocation-free entry point takes at most 128 sequences per call");
    for (int b = 0; b < B; ++b)
        if (pos[b] < 0 || pos[b] >= c->cfg.seq_len) return fail(c, GGR_ERR_RANGE, "position outside the cache");
    const size_t part_cap = (GGR_STATIC_SCRATCH_BYTES - GGR_STATIC_TICKET_BYTES) / sizeof(float);
    const size_t per_split = (size_t)B * c->kv.Hq * (c->D + 2);
    const size_t tickets = (size_t)B * c->kv.Hkv;

    Items it{};
    it.mode = 0;
    it.seq0 = 0;
    it.n = B;
    for (int i = 0; i < B; ++i) it.pos[i] = pos[i];
    AttnArgs a{};
    a.kv = c->kv;
    a.items = it;
    a.vis = visibility(c, layer);
    a.layer = layer;
    a.q = q_dev;
    a.score_scale = (c->cfg.scale_mode == GGR_SCALE_SCORE ? c->attn_scale : 1.0f) * kLog2e;
    a.out = out_dev;
    a.partial_out = nullptr;
    a.shard_count = c->shard_count;
    a.err = c->d_err;
    DecodePlan dp = decode_plan(c, true);
    const int t_max = t_max_of(c, layer, pos, B);
    // The split count comes first: a call that runs unsplit (a short context, or so many (sequence, kv head)
    // groups that they fill the GPU by themselves) needs no scratch and is never rejected for its size.
    a.n_split = plan_splits(c, dp, B, t_max, c->cfg.max_splits);
    const bool mma = dp.mma, tma = dp.tma, tile = dp.tile;
    SimtPlan p = dp.p;
    if (tile) p.smem = dp.smem;
    size_t smem = dp.smem;
    a.stage_bytes = p.stage_bytes;
    a.tile_stages = dp.tp.nst;
    if (a.n_split > 1) {
        const size_t fit = part_cap / per_split;  // splits the array can hold
        if (fit < 2 || tickets * sizeof(unsigned) > GGR_STATIC_TICKET_BYTES) {
            char buf[200];
            snprintf(buf, sizeof buf,
                     "static scratch too small: B*n_heads*(head_dim+2) = %zu floats per split, the 8 MiB array holds two "
                     "splits only up to %zu", per_split, part_cap / 2);
            return fail(c, GGR_ERR_RANGE, buf);
        }
        a.n_split = (int)std::min<size_t>((size_t)a.n_split, fit);
    }
    unsigned char* scratch = nullptr;
    if ((rc = static_scratch(c, &scratch))) return rc;
    c->last_splits = a.n_split;
    const size_t merge_smem = split_merge_smem_bytes(c, a.n_split);
    smem = std::max(smem, merge_smem);
    p.smem = std::max(p.smem, merge_smem);
    if (a.n_split > 1) {
        a.counters = reinterpret_cast<unsigned*>(scratch);
        a.part = reinterpret_cast<float*>(scratch + GGR_STATIC_TICKET_BYTES);
        // the array keeps whatever the previous call (of any context) left: tickets must start at zero
        CUDA_TRY(c, cudaMemsetAsync(a.counters, 0, tickets * sizeof(unsigned), c->stream));
    }
    dim3 grid(a.n_split, c->kv.Hkv, B);
    if (mma) {
        int e;
        {
            LaunchTimer t(c, 0);
            e = tma ? launch_mma_tma_decode(c->tmK16, c->tmV16, a, grid, smem, c->smem_optin, c->cfg.device, c->stream)
                    : launch_mma_decode(a, grid, smem, c->smem_optin, c->cfg.device, c->stream);
        }
        if (e != 0) return fail(c, GGR_ERR_CUDA, std::string("mma decode launch: ") + cudaGetErrorString((cudaError_t)e));
        c->launches++;
        return GGR_OK;
    }
    if (tile) {
        int e;
        {
            LaunchTimer t(c, 0);
            e = launch_tile_decode(a, grid, smem, c->smem_optin, c->cfg.device, c->stream);
        }
        if (e != 0) return fail(c, GGR_ERR_CUDA, std::string("tile decode launch: ") + cudaGetErrorString((cudaError_t)e));
        c->launches++;
        return GGR_OK;
    }
    return launch_simt(c, a, grid, p);
}

#ifdef GGR_TC_TRACE
// diagnostic builds only: device buffer of 32 int64 cycle counters written by CTA 0 of the prefill kernel
extern "C" void ggr_attn_debug_set_trace(long long* device_ptr) { g_tc_trace = device_ptr; }
#endif

// ---- fused exchange of KV-sequence shards -----------------------------------------------------------

namespace {
size_t x_slot_floats(const ggr_attn_ctx* c) { return (size_t)c->x_max_b * c->kv.Hq * (c->D + 2); }
size_t x_flag_bytes() { return 256; }
size_t x_total_bytes(const ggr_attn_ctx* c) {
    return x_flag_bytes() + 2 * (size_t)c->cfg.n_ranks * x_slot_floats(c) * sizeof(float);
}
}  // namespace

extern "C" int ggr_attn_exchange_create(ggr_attn_ctx* c, int32_t max_B, void** local_base, unsigned char* ipc_handle) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (c->cfg.shard_mode != GGR_SHARD_KV_SEQUENCE) return fail(c, GGR_ERR_INVALID, "the exchange belongs to a KV-sequence shard");
    if (c->cfg.n_ranks < 1 || c->cfg.n_ranks > kMaxPeers || c->cfg.rank < 0 || c->cfg.rank >= c->cfg.n_ranks)
        return fail(c, GGR_ERR_INVALID, "the exchange supports 1 to 8 ranks");
    if (max_B <= 0 || max_B > c->cfg.max_batch || max_B > kMaxArgItems) return fail(c, GGR_ERR_RANGE, "exchange batch out of range");
    if (c->x_local) return fail(c, GGR_ERR_INVALID, "the exchange buffer already exists");
    c->x_max_b = max_B;
    const size_t bytes = x_total_bytes(c);
    if (cudaMalloc((void**)&c->x_local, bytes) != cudaSuccess || cudaMalloc((void**)&c->d_done, sizeof(unsigned)) != cudaSuccess) {
        cudaGetLastError();
        return fail(c, GGR_ERR_ALLOC, "unable to allocate the exchange buffer");
    }
    CUDA_TRY(c, cudaMemset(c->x_local, 0, bytes));
    CUDA_TRY(c, cudaMemset(c->d_done, 0, sizeof(unsigned)));
    c->x_peer[c->cfg.rank] = c->x_local;
    if (local_base) *local_base = c->x_local;
    if (ipc_handle) {
        cudaIpcMemHandle_t h;
        CUDA_TRY(c, cudaIpcGetMemHandle(&h, c->x_local));
        static_assert(sizeof(h) == 64, "IPC handle size");
        std::memcpy(ipc_handle, &h, 64);
    }
    return GGR_OK;
}

extern "C" int ggr_attn_exchange_connect(ggr_attn_ctx* c, const unsigned char* ipc_handles, void* const* same_process_ptrs) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (!c->x_local) return fail(c, GGR_ERR_INVALID, "create the exchange buffer first");
    if (!ipc_handles && !same_process_ptrs) return fail(c, GGR_ERR_INVALID, "no peer buffers given");
    for (int r = 0; r < c->cfg.n_ranks; ++r) {
        if (r == c->cfg.rank) continue;
        if (same_process_ptrs && same_process_ptrs[r]) {
            c->x_peer[r] = static_cast<unsigned char*>(same_process_ptrs[r]);
            continue;
        }
        if (!ipc_handles) return fail(c, GGR_ERR_INVALID, "missing peer buffer");
        cudaIpcMemHandle_t h;
        std::memcpy(&h, ipc_handles + (size_t)r * 64, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail(c, GGR_ERR_COMM, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
        c->x_peer[r] = static_cast<unsigned char*>(p);
        c->x_opened[r] = true;
    }
    c->x_connected = true;
    return GGR_OK;
}

namespace {

// send half: fused decode over the local slab, states stored into every rank's receive slot, flag raised
int exchange_send(ggr_attn_ctx* c, int layer, const int32_t* pos, int B, const float* q, const float* k, const float* v,
                  int ptr_kind) {
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!c->x_connected) return fail(c, GGR_ERR_INVALID, "connect the exchange buffers first");
    if (B <= 0 || B > c->x_max_b) return fail(c, GGR_ERR_RANGE, "batch larger than the exchange buffer");
    if (!pos || !q || !k || !v) return fail(c, GGR_ERR_INVALID, "null buffer");
    for (int b = 0; b < B; ++b)
        if (pos[b] < 0 || pos[b] >= c->cfg.seq_len) return fail(c, GGR_ERR_RANGE, "position outside the cache");
    const size_t qb = (size_t)B * c->q_dim * sizeof(float), kb = (size_t)B * c->kv_dim * sizeof(float);
    const void *dq, *dk, *dv;
    if ((rc = stage_in(c, 0, q, qb, ptr_kind, &dq))) return rc;
    if ((rc = stage_in(c, 1, k, kb, ptr_kind, &dk))) return rc;
    if ((rc = stage_in(c, 2, v, kb, ptr_kind, &dv))) return rc;
    if ((rc = ensure(c, &c->d_qrot, &c->qrot_cap, (size_t)B * c->q_dim))) return rc;
    int in_bf16 = 0;
    if ((rc = apply_fixups(c, layer, B, &dq, &dk, &dv, &in_bf16))) return rc;
    const int n = c->cfg.n_ranks, me = c->cfg.rank;
    // the step counter moves only once the kernel is in the stream: a send that fails on the host leaves the
    // ranks' counters in agreement
    const int epoch = c->x_epoch + 1;
    const size_t slot = x_slot_floats(c), parity_off = (size_t)(epoch & 1) * n * slot;
    PeerExchange px{};
    px.enabled = 1;
    px.n_ranks = n;
    px.rank = me;
    px.epoch = epoch;
    px.done_counter = c->d_done;
    px.groups_total = B * c->kv.Hkv;
    for (int r = 0; r < n; ++r) {
        px.slot[r] = reinterpret_cast<float*>(c->x_peer[r] + x_flag_bytes()) + parity_off + (size_t)me * slot;
        px.flag[r] = reinterpret_cast<int*>(c->x_peer[r]) + me;
    }
    Items it{};
    it.mode = 0;
    it.seq0 = 0;
    it.n = B;
    for (int i = 0; i < B; ++i) it.pos[i] = pos[i];
    const RawDecodeInputs raw{static_cast<const float*>(dq), static_cast<const float*>(dk), static_cast<const float*>(dv)};
    rc = launch_attention(c, layer, it, t_max_of(c, layer, pos, B), c->d_qrot, nullptr, nullptr, true, &raw, &px);
    if (rc == GGR_OK) c->x_epoch = epoch;
    return rc;
}


// receive half: bounded wait for every rank's flag of the current step, then the merge
// `after_own_send`: the merge kernel is enqueued right behind this rank's own send kernel. It may then start while
// that kernel is still running (programmatic dependent launch: the send kernels signal launch_dependents as soon as
// all their CTAs are resident), so its launch latency and its wait for the peers overlap the local decode instead of
// following it. The merge never reads anything but what the flags guard, so it needs no grid dependency wait.
int exchange_receive(ggr_attn_ctx* c, int B, float* out, int ptr_kind, bool after_own_send = false) {
    if (!c->x_connected || c->x_epoch == 0) return fail(c, GGR_ERR_INVALID, "nothing was sent on this exchange yet");
    if (B <= 0 || B > c->x_max_b || !out) return fail(c, GGR_ERR_INVALID, "invalid receive arguments");
    const size_t qb = (size_t)B * c->q_dim * sizeof(float);
    float* dout = out;
    int rc;
    if (ptr_kind == GGR_PTR_HOST) {
        if ((rc = ensure(c, &c->d_stage[3], &c->stage_cap[3], qb))) return rc;
        dout = reinterpret_cast<float*>(c->d_stage[3]);
    }
    const int n = c->cfg.n_ranks, epoch = c->x_epoch;
    const size_t slot = x_slot_floats(c), parity_off = (size_t)(epoch & 1) * n * slot;
    {
        LaunchTimer t(c, 2);
        const float* parts = reinterpret_cast<const float*>(c->x_local + x_flag_bytes()) + parity_off;
        const int* flags = reinterpret_cast<const int*>(c->x_local);
        if (after_own_send && !c->timing) {
            cudaLaunchConfig_t lc{};
            lc.gridDim = dim3((c->kv.Hq + kCombineHeads - 1) / kCombineHeads, B);
            lc.blockDim = dim3(kCombineHeads * 32);
            lc.dynamicSmemBytes = 0;
            lc.stream = c->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            lc.attrs = attr;
            lc.numAttrs = 1;
            CUDA_TRY(c, cudaLaunchKernelEx(&lc, combine_exchange_kernel, parts, flags, epoch, n, (int64_t)slot, (int)c->kv.Hq,
                                           (int)c->D, dout, c->d_err, c->x_wait_ns, (const float*)nullptr, 0));
        } else {
            combine_exchange_kernel<<<dim3((c->kv.Hq + kCombineHeads - 1) / kCombineHeads, B), kCombineHeads * 32, 0, c->stream>>>(parts, flags, epoch, n, (int64_t)slot, c->kv.Hq,
                                                                              c->D, dout, c->d_err, c->x_wait_ns, nullptr, 0);
        }
    }
    CUDA_TRY(c, cudaGetLastError());
    c->launches++;
    if (ptr_kind == GGR_PTR_HOST) {
        CUDA_TRY(c, cudaMemcpyAsync(out, dout, qb, cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        return take_device_error(c, "a peer's partial states did not arrive in time");
    }
    return GGR_OK;
}

}  // namespace

extern "C" int ggr_attn_exchange_send(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                                      const float* k, const float* v, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = exchange_send(c, layer, pos, B, q, k, v, ptr_kind);
    if (rc == GGR_OK && ptr_kind == GGR_PTR_HOST) CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return rc;
}

extern "C" int32_t ggr_attn_exchange_epoch(const ggr_attn_ctx* c) { return c ? c->x_epoch : 0; }

extern "C" int ggr_attn_exchange_resync(ggr_attn_ctx* c, int32_t epoch) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (!c->x_connected) return fail(c, GGR_ERR_INVALID, "connect the exchange buffers first");
    if (epoch < c->x_epoch) return fail(c, GGR_ERR_INVALID, "the step counter only moves forward: pass the maximum over all ranks");
    // nothing of an abandoned step may still be in flight when the counters are realigned
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    if (c->h_err) *c->h_err = 0;
    // a send that never completed its groups leaves a partial count behind
    CUDA_TRY(c, cudaMemset(c->d_done, 0, sizeof(unsigned)));
    c->x_epoch = epoch;
    return GGR_OK;
}

extern "C" int ggr_attn_exchange_receive(ggr_attn_ctx* c, int32_t B, float* out, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    return exchange_receive(c, B, out, ptr_kind);
}

extern "C" int ggr_attn_decode_exchange(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                                        const float* k, const float* v, float* out, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = exchange_send(c, layer, pos, B, q, k, v, ptr_kind);
    if (rc) return rc;
    return exchange_receive(c, B, out, ptr_kind, true);
}

// ---- per-layer pre-attention fixups ----------------------------------------------------------------------

extern "C" int ggr_attn_set_layer_fixups(ggr_attn_ctx* c, int32_t layer, const float* q_bias, const float* k_bias,
                                         const float* v_bias, const float* q_norm, const float* k_norm, float eps) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if ((q_bias || k_bias || v_bias) && !(q_bias && k_bias && v_bias))
        return fail(c, GGR_ERR_INVALID, "q, k and v biases come together");
    if ((q_norm || k_norm) && !(q_norm && k_norm)) return fail(c, GGR_ERR_INVALID, "q and k norm weights come together");
    CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    c->fixups.resize(c->cfg.n_layers);
    auto& f = c->fixups[layer];
    for (float** p : {&f.q_bias, &f.k_bias, &f.v_bias, &f.q_norm, &f.k_norm}) {
        cudaFree(*p);
        *p = nullptr;
    }
    auto upload = [&](float** dst, const float* src, size_t n) -> int {
        if (!src) return GGR_OK;
        if (cudaMalloc((void**)dst, n * sizeof(float)) != cudaSuccess) return fail(c, GGR_ERR_ALLOC, "unable to allocate fixups");
        CUDA_TRY(c, cudaMemcpy(*dst, src, n * sizeof(float), cudaMemcpyHostToDevice));
        return GGR_OK;
    };
    if ((rc = upload(&f.q_bias, q_bias, c->q_dim))) return rc;
    if ((rc = upload(&f.k_bias, k_bias, c->kv_dim))) return rc;
    if ((rc = upload(&f.v_bias, v_bias, c->kv_dim))) return rc;
    if ((rc = upload(&f.q_norm, q_norm, c->D))) return rc;
    if ((rc = upload(&f.k_norm, k_norm, c->D))) return rc;
    f.eps = eps;
    return GGR_OK;
}


// ---- projections either side of the path -----------------------------------------------------------------------------

struct ggr_weights {
    int device = 0, wtype = 0, rows = 0, cols = 0;
    void* d_main = nullptr;            // F32 / BF16 values, or the Q8_0 code plane
    __half* d_scales = nullptr;        // Q8_0 block scales [rows][cols / 32]; Q4_K: (scale, min) byte pairs per 32 weights
    __half2* d_dm = nullptr;           // Q4_K: (d, dmin) per super-block [rows][cols / 256]
    float* d_scales_f32 = nullptr;     // Q6_K: d * scale per 16 weights [rows][cols / 16]
    __nv_bfloat16* d_bf16 = nullptr;   // bf16 image for the tensor-core kernel (d_main itself for BF16)
    CUtensorMap tmB;                   // [rows][cols] bf16, box 64 x 256
    bool have_tmap = false;
};

namespace {

float half_bits_to_float(uint16_t h) {  // IEEE half -> single (src/engine/io/gguf.rs:27-52)
    const uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
    int exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x03ffu, bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            while ((mant & 0x0400u) == 0) {
                mant <<= 1;
                exp -= 1;
            }
            exp += 1;
            mant &= ~0x0400u;
            bits = sign | ((uint32_t)(exp + 112) << 23) | (mant << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (mant << 13);
    } else {
        bits = sign | ((uint32_t)(exp + 112) << 23) | (mant << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

uint16_t float_to_bf16_bits(float f) {  // round to nearest even (src/engine/io/gguf.rs:107-116)
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// xout [n][w->rows] = x [n][w->cols] W^T, device pointers
void fill_gemv(GemvArgs& a, const ggr_weights* w, const float* x, int n, float* out, int ld_out, int sanitize) {
    a.w = w->d_main;
    a.scales = w->d_scales;
    a.dm = w->d_dm;
    a.scales_f32 = w->d_scales_f32;
    a.rows = w->rows;
    a.cols = w->cols;
    a.x = x;
    a.n = n;
    a.out = out;
    a.ld_out = ld_out;
    a.sanitize = sanitize;
}

int matmul_device(ggr_attn_ctx* c, const ggr_weights* w, const float* x, int n, float* out, __nv_bfloat16* out_h, int ld_out,
                  int sanitize) {
    if (w->device != c->cfg.device) return fail(c, GGR_ERR_INVALID, "the weights live on another device than the context");
    if (n <= 16 && !out_h && w->cols <= kGemvMaxCols) {
        GemvArgs a{};
        fill_gemv(a, w, x, n, out, ld_out, sanitize);
        {
            LaunchTimer t(c, 3);
            CUDA_TRY(c, launch_gemv(w->wtype, a, c->cfg.device, c->sm_count, c->stream));
        }
        c->launches++;
        return GGR_OK;
    }
    if (!w->have_tmap) return fail(c, GGR_ERR_UNSUPPORTED, "no tensor map for these weights (driver entry point missing)");
    int rc = ensure(c, &c->d_pact, &c->pact_cap, (size_t)n * w->cols);
    if (rc) return rc;
    const size_t elems = (size_t)n * w->cols;
    proj_to_bf16_kernel<<<(unsigned)std::min<size_t>(2048, (elems / 4 + 255) / 256 + 1), 256, 0, c->stream>>>(x, c->d_pact, elems);
    CUDA_TRY(c, cudaGetLastError());
    c->launches++;
    CUtensorMap tmA;
    if (!make_tmap_bf16(&tmA, c->d_pact, (uint64_t)w->cols, (uint64_t)n, kGemmBM))
        return fail(c, GGR_ERR_CUDA, "cuTensorMapEncodeTiled failed for the activation rows");
    GemmArgs g{};
    g.m = n;
    g.N = w->rows;
    g.K = w->cols;
    g.out = out;
    g.out_h = out_h;
    g.ld_out = ld_out;
    g.sanitize = sanitize;
    g.err = c->d_err;
    {
        LaunchTimer t(c, 3);
        CUDA_TRY(c, launch_gemm(tmA, w->tmB, g, c->cfg.device, c->stream));
    }
    c->launches++;
    return GGR_OK;
}

int check_layer_weights(ggr_attn_ctx* c, const ggr_weights* wq, const ggr_weights* wk, const ggr_weights* wv,
                        const ggr_weights* wo) {
    if (!wq || !wk || !wv || !wo) return fail(c, GGR_ERR_INVALID, "null weights");
    if (wq->rows != c->q_dim || wk->rows != c->kv_dim || wv->rows != c->kv_dim || wo->cols != c->q_dim ||
        wk->cols != wq->cols || wv->cols != wq->cols)
        return fail(c, GGR_ERR_INVALID, "projection shapes do not match the attention shape (wq [q_dim][dim], wk / wv "
                                        "[kv_dim][dim], wo [dim][q_dim])");
    return GGR_OK;
}

}  // namespace

extern "C" int ggr_weights_upload(int32_t device, int32_t wtype, int32_t rows, int32_t cols, const void* host_data,
                                  ggr_weights** out) {
    auto bad = [&](int st, const char* msg) {
        g_create_err = msg;
        return st;
    };
    if (!out || !host_data) return bad(GGR_ERR_INVALID, "null argument");
    *out = nullptr;
    if (wtype < GGR_W_F32 || wtype > GGR_W_Q6_K) return bad(GGR_ERR_INVALID, "unknown weight type");
    const int col_unit = (wtype == GGR_W_Q4_K || wtype == GGR_W_Q6_K) ? 256 : (wtype == GGR_W_Q8_0 ? 32 : 8);
    if (rows <= 0 || cols <= 0 || rows % 8 != 0 || cols % col_unit != 0)
        return bad(GGR_ERR_UNSUPPORTED, "rows must be a multiple of 8, cols of 8 (32 for Q8_0, 256 for Q4_K and Q6_K)");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return bad(GGR_ERR_CUDA, "no such CUDA device");
    DeviceGuard guard(device);
    ggr_weights* w = new ggr_weights();
    w->device = device;
    w->wtype = wtype;
    w->rows = rows;
    w->cols = cols;
    const size_t n = (size_t)rows * cols;
    auto fail_up = [&](const char* msg) {
        cudaGetLastError();
        ggr_weights_free(w);
        return bad(GGR_ERR_ALLOC, msg);
    };
    std::vector<uint16_t> image;  // bf16 image of F32 / Q8_0 weights
    if (wtype == GGR_W_BF16) {
        if (cudaMalloc(&w->d_main, n * 2) != cudaSuccess) return fail_up("unable to allocate the weights");
        if (cudaMemcpy(w->d_main, host_data, n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return fail_up("weight upload failed");
        w->d_bf16 = static_cast<__nv_bfloat16*>(w->d_main);
    } else if (wtype == GGR_W_F32) {
        if (cudaMalloc(&w->d_main, n * 4) != cudaSuccess) return fail_up("unable to allocate the weights");
        if (cudaMemcpy(w->d_main, host_data, n * 4, cudaMemcpyHostToDevice) != cudaSuccess) return fail_up("weight upload failed");
        image.resize(n);
        const float* src = static_cast<const float*>(host_data);
        for (size_t i = 0; i < n; ++i) image[i] = float_to_bf16_bits(src[i]);
    } else if (wtype == GGR_W_Q4_K) {
        // 144-byte super-blocks -> a nibble plane [rows][cols / 2] in which every 32 weights of one (scale, min) pair
        // are 16 contiguous bytes (byte i = weight i | weight i + 16 << 4), a plane of (scale, min) byte pairs per 32
        // weights and a plane of (d, dmin) per 256 (get_scale_min_k4, src/engine/kernels/quant.rs:118-126)
        const size_t nsb = n / 256, nb32 = n / 32;
        std::vector<uint8_t> codes(n / 2);
        std::vector<uint16_t> sm(nb32);
        std::vector<uint32_t> dm(nsb);
        image.resize(n);
        const uint8_t* src = static_cast<const uint8_t*>(host_data);
        for (size_t b = 0; b < nsb; ++b) {
            const uint8_t* blk = src + b * 144;
            const uint16_t dh = (uint16_t)(blk[0] | (blk[1] << 8)), mh = (uint16_t)(blk[2] | (blk[3] << 8));
            dm[b] = (uint32_t)dh | ((uint32_t)mh << 16);
            const float d = half_bits_to_float(dh), dmin = half_bits_to_float(mh);
            const uint8_t* sc = blk + 4;
            const uint8_t* qs = blk + 16;
            for (int j = 0; j < 8; ++j) {
                int s6, m6;
                if (j < 4) {
                    s6 = sc[j] & 63;
                    m6 = sc[j + 4] & 63;
                } else {
                    s6 = (sc[j + 4] & 0x0f) | ((sc[j - 4] >> 6) << 4);
                    m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
                }
                sm[b * 8 + j] = (uint16_t)(s6 | (m6 << 8));
                const float d1 = d * (float)s6, m1f = dmin * (float)m6;
                uint8_t q[32];
                for (int l = 0; l < 32; ++l) q[l] = (j & 1) ? (uint8_t)(qs[(j >> 1) * 32 + l] >> 4) : (uint8_t)(qs[(j >> 1) * 32 + l] & 0x0f);
                for (int l = 0; l < 16; ++l) codes[(b * 8 + j) * 16 + l] = (uint8_t)(q[l] | (q[l + 16] << 4));
                for (int l = 0; l < 32; ++l) image[b * 256 + j * 32 + l] = float_to_bf16_bits(d1 * (float)q[l] - m1f);
            }
        }
        if (cudaMalloc(&w->d_main, n / 2) != cudaSuccess || cudaMalloc((void**)&w->d_scales, nb32 * 2) != cudaSuccess ||
            cudaMalloc((void**)&w->d_dm, nsb * 4) != cudaSuccess)
            return fail_up("unable to allocate the weights");
        if (cudaMemcpy(w->d_main, codes.data(), n / 2, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(w->d_scales, sm.data(), nb32 * 2, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(w->d_dm, dm.data(), nsb * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return fail_up("weight upload failed");
    } else if (wtype == GGR_W_Q6_K) {
        // 210-byte super-blocks -> the weights as int8 codes (q - 32) [rows][cols] and one f32 scale d * sc per 16
        // weights [rows][cols / 16] (weight e of a super-block uses scale e / 16: dequantize_row_q6_k,
        // src/engine/kernels/quant.rs:484-517)
        const size_t nsb = n / 256;
        std::vector<int8_t> codes(n);
        std::vector<float> sc16(n / 16);
        image.resize(n);
        const uint8_t* src = static_cast<const uint8_t*>(host_data);
        for (size_t b = 0; b < nsb; ++b) {
            const uint8_t* blk = src + b * 210;
            const float d = half_bits_to_float((uint16_t)(blk[208] | (blk[209] << 8)));
            const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
            for (int g16 = 0; g16 < 16; ++g16) sc16[b * 16 + g16] = d * (float)sc[g16];
            for (int half = 0; half < 2; ++half) {
                const uint8_t* ql = blk + 64 * half;
                const uint8_t* qh = blk + 128 + 32 * half;
                for (int l = 0; l < 32; ++l) {
                    const int q[4] = {(int)((ql[l] & 0x0f) | ((qh[l] & 0x03) << 4)) - 32,
                                      (int)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 0x03) << 4)) - 32,
                                      (int)((ql[l] >> 4) | (((qh[l] >> 4) & 0x03) << 4)) - 32,
                                      (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 0x03) << 4)) - 32};
                    for (int k = 0; k < 4; ++k) {
                        const size_t e = b * 256 + 128 * half + 32 * k + l;
                        codes[e] = (int8_t)q[k];
                        image[e] = float_to_bf16_bits(sc16[e / 16] * (float)q[k]);
                    }
                }
            }
        }
        if (cudaMalloc(&w->d_main, n) != cudaSuccess || cudaMalloc((void**)&w->d_scales_f32, (n / 16) * 4) != cudaSuccess)
            return fail_up("unable to allocate the weights");
        if (cudaMemcpy(w->d_main, codes.data(), n, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(w->d_scales_f32, sc16.data(), (n / 16) * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return fail_up("weight upload failed");
    } else {
        // 34-byte blocks -> a code plane [rows][cols] and a scale plane [rows][cols / 32]
        const size_t nb = n / 32;
        std::vector<int8_t> codes(n);
        std::vector<uint16_t> scales(nb);
        image.resize(n);
        const uint8_t* src = static_cast<const uint8_t*>(host_data);
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = src + b * 34;
            scales[b] = (uint16_t)(blk[0] | (blk[1] << 8));
            const float d = half_bits_to_float(scales[b]);
            for (int j = 0; j < 32; ++j) {
                const int8_t q = (int8_t)blk[2 + j];
                codes[b * 32 + j] = q;
                image[b * 32 + j] = float_to_bf16_bits((float)q * d);
            }
        }
        if (cudaMalloc(&w->d_main, n) != cudaSuccess || cudaMalloc((void**)&w->d_scales, nb * 2) != cudaSuccess)
            return fail_up("unable to allocate the weights");
        if (cudaMemcpy(w->d_main, codes.data(), n, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(w->d_scales, scales.data(), nb * 2, cudaMemcpyHostToDevice) != cudaSuccess)
            return fail_up("weight upload failed");
    }
    if (!image.empty()) {
        if (cudaMalloc((void**)&w->d_bf16, n * 2) != cudaSuccess) return fail_up("unable to allocate the bf16 weight image");
        if (cudaMemcpy(w->d_bf16, image.data(), n * 2, cudaMemcpyHostToDevice) != cudaSuccess) return fail_up("weight upload failed");
    }
    w->have_tmap = make_tmap_bf16(&w->tmB, w->d_bf16, (uint64_t)cols, (uint64_t)rows, kGemmBN);
    g_create_err.clear();
    *out = w;
    return GGR_OK;
}

extern "C" void ggr_weights_free(ggr_weights* w) {
    if (!w) return;
    DeviceGuard guard(w->device);
    if (w->d_bf16 && w->d_bf16 != w->d_main) cudaFree(w->d_bf16);
    cudaFree(w->d_main);
    cudaFree(w->d_scales);
    cudaFree(w->d_dm);
    cudaFree(w->d_scales_f32);
    delete w;
}

extern "C" int ggr_proj_matmul(ggr_attn_ctx* c, const ggr_weights* w, const float* x, int32_t n, float* xout, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    if (!w || !x || !xout || n <= 0) return fail(c, GGR_ERR_INVALID, "invalid matmul arguments");
    const size_t in_elems = (size_t)n * w->cols, out_elems = (size_t)n * w->rows;
    const float* dx = x;
    float* dout = xout;
    int rc;
    if (ptr_kind == GGR_PTR_HOST) {
        if ((rc = ensure(c, &c->d_px, &c->px_cap, in_elems))) return rc;
        if ((rc = ensure(c, &c->d_pout, &c->pout_cap, out_elems))) return rc;
        CUDA_TRY(c, cudaMemcpyAsync(c->d_px, x, in_elems * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        dx = c->d_px;
        dout = c->d_pout;
    }
    if ((rc = matmul_device(c, w, dx, n, dout, nullptr, w->rows, 0))) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        CUDA_TRY(c, cudaMemcpyAsync(xout, dout, out_elems * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        return take_device_error(c, "a bounded wait inside the matmul kernel ran out");
    }
    return GGR_OK;
}

extern "C" int ggr_attn_layer_decode(ggr_attn_ctx* c, int32_t layer, const int32_t* pos, int32_t B, const float* xb,
                                     const ggr_weights* wq, const ggr_weights* wk, const ggr_weights* wv,
                                     const ggr_weights* wo, float* xb2, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!pos || !xb || !xb2) return fail(c, GGR_ERR_INVALID, "null buffer");
    if (B <= 0 || B > c->cfg.max_batch) return fail(c, GGR_ERR_RANGE, "batch larger than max_batch");
    if (c->cfg.shard_mode != GGR_SHARD_NONE) return fail(c, GGR_ERR_UNSUPPORTED, "not available on a KV-sequence shard");
    if ((rc = check_layer_weights(c, wq, wk, wv, wo))) return rc;
    const int dim = wq->cols, dim_out = wo->rows;
    const size_t qkv = (size_t)c->q_dim + 2 * c->kv_dim;
    const float* dx = xb;
    float* dout = xb2;
    if ((rc = ensure(c, &c->d_pqkv, &c->pqkv_cap, (size_t)B * qkv))) return rc;
    if ((rc = ensure(c, &c->d_patt, &c->patt_cap, (size_t)B * c->q_dim))) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        const size_t in_bytes = (size_t)B * dim * sizeof(float), out_bytes = (size_t)B * dim_out * sizeof(float);
        if ((rc = ensure_pinned(c, in_bytes, out_bytes))) return rc;
        if ((rc = ensure(c, &c->d_pout, &c->pout_cap, (size_t)B * dim_out))) return rc;
        std::memcpy(c->h_pin, xb, in_bytes);
        CUDA_TRY(c, cudaMemcpyAsync(c->d_pin_in, c->h_pin, in_bytes, cudaMemcpyHostToDevice, c->stream));
        dx = reinterpret_cast<const float*>(c->d_pin_in);
        dout = c->d_pout;
    }
    float* dq = c->d_pqkv;
    float* dk = dq + (size_t)B * c->q_dim;
    float* dv = dk + (size_t)B * c->kv_dim;
    if (B <= 16 && wq->cols <= kGemvMaxCols && wk->wtype == wq->wtype && wv->wtype == wq->wtype) {
        // the three projections read the same rows: one launch over the rows of wq, wk and wv
        GemvArgs a{};
        fill_gemv(a, wq, dx, B, dq, c->q_dim, 0);
        const ggr_weights* extra[2] = {wk, wv};
        float* outs[2] = {dk, dv};
        a.n_extra = 2;
        a.rows_all = wq->rows + wk->rows + wv->rows;
        for (int i = 0; i < 2; ++i) {
            a.w_x[i] = extra[i]->d_main;
            a.scales_x[i] = extra[i]->d_scales;
            a.dm_x[i] = extra[i]->d_dm;
            a.scales_f32_x[i] = extra[i]->d_scales_f32;
            a.rows_x[i] = extra[i]->rows;
            a.out_x[i] = outs[i];
            a.ld_out_x[i] = c->kv_dim;
        }
        {
            LaunchTimer t(c, 3);
            CUDA_TRY(c, launch_gemv(wq->wtype, a, c->cfg.device, c->sm_count, c->stream));
        }
        c->launches++;
    } else {
        if ((rc = matmul_device(c, wq, dx, B, dq, nullptr, c->q_dim, 0))) return rc;
        if ((rc = matmul_device(c, wk, dx, B, dk, nullptr, c->kv_dim, 0))) return rc;
        if ((rc = matmul_device(c, wv, dx, B, dv, nullptr, c->kv_dim, 0))) return rc;
    }
    if ((rc = decode_common(c, layer, pos, B, dq, dk, dv, c->d_patt, nullptr, GGR_PTR_DEVICE))) return rc;
    if ((rc = matmul_device(c, wo, c->d_patt, B, dout, nullptr, dim_out, 1))) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        const size_t out_bytes = (size_t)B * dim_out * sizeof(float);
        unsigned char* h_out = c->h_pin + (c->pin_cap - out_bytes);
        CUDA_TRY(c, cudaMemcpyAsync(h_out, dout, out_bytes, cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        std::memcpy(xb2, h_out, out_bytes);
        return take_device_error(c, "a bounded wait inside a kernel ran out");
    }
    return GGR_OK;
}

extern "C" int ggr_attn_layer_prefill(ggr_attn_ctx* c, int32_t layer, int32_t seq, int32_t base_pos, int32_t m,
                                      const float* xb, const ggr_weights* wq, const ggr_weights* wk, const ggr_weights* wv,
                                      const ggr_weights* wo, float* xb2, int32_t ptr_kind) {
    if (!c) return GGR_ERR_INVALID;
    DeviceGuard guard(c->cfg.device);
    int rc = check_layer(c, layer);
    if (rc) return rc;
    if (!xb || !xb2 || m <= 0) return fail(c, GGR_ERR_INVALID, "invalid prefill arguments");
    if ((rc = check_layer_weights(c, wq, wk, wv, wo))) return rc;
    const int dim = wq->cols, dim_out = wo->rows;
    const size_t qkv = (size_t)c->q_dim + 2 * c->kv_dim;
    const float* dx = xb;
    float* dout = xb2;
    if ((rc = ensure(c, &c->d_patt, &c->patt_cap, (size_t)m * c->q_dim))) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        if ((rc = ensure(c, &c->d_px, &c->px_cap, (size_t)m * dim))) return rc;
        if ((rc = ensure(c, &c->d_pout, &c->pout_cap, (size_t)m * dim_out))) return rc;
        CUDA_TRY(c, cudaMemcpyAsync(c->d_px, xb, (size_t)m * dim * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        dx = c->d_px;
        dout = c->d_pout;
    }
    // Chunks on the tensor-core kernel hand q / k / v on in bf16 when the cache is bf16 (what the tcgen05 attention
    // kernel reads anyway); the weight-streaming kernel and the other cache formats stay in f32.
    const bool fixups = (size_t)layer < c->fixups.size() && c->fixups[layer].any();
    const bool half_out = m > 16 && c->kv.fmt == KV_BF16 && !fixups;
    if (half_out) {
        if ((rc = ensure(c, &c->d_pqkv_h, &c->pqkv_h_cap, (size_t)m * qkv))) return rc;
        __nv_bfloat16* hq = c->d_pqkv_h;
        __nv_bfloat16* hk = hq + (size_t)m * c->q_dim;
        __nv_bfloat16* hv = hk + (size_t)m * c->kv_dim;
        if ((rc = matmul_device(c, wq, dx, m, nullptr, hq, c->q_dim, 0))) return rc;
        if ((rc = matmul_device(c, wk, dx, m, nullptr, hk, c->kv_dim, 0))) return rc;
        if ((rc = matmul_device(c, wv, dx, m, nullptr, hv, c->kv_dim, 0))) return rc;
        rc = prefill_common(c, layer, seq, base_pos, m, hq, hk, hv, GGR_DTYPE_BF16, c->d_patt, GGR_PTR_DEVICE, false);
    } else {
        if ((rc = ensure(c, &c->d_pqkv, &c->pqkv_cap, (size_t)m * qkv))) return rc;
        float* dq = c->d_pqkv;
        float* dk = dq + (size_t)m * c->q_dim;
        float* dv = dk + (size_t)m * c->kv_dim;
        if ((rc = matmul_device(c, wq, dx, m, dq, nullptr, c->q_dim, 0))) return rc;
        if ((rc = matmul_device(c, wk, dx, m, dk, nullptr, c->kv_dim, 0))) return rc;
        if ((rc = matmul_device(c, wv, dx, m, dv, nullptr, c->kv_dim, 0))) return rc;
        rc = prefill_common(c, layer, seq, base_pos, m, dq, dk, dv, GGR_DTYPE_F32, c->d_patt, GGR_PTR_DEVICE, false);
    }
    if (rc) return rc;
    if ((rc = matmul_device(c, wo, c->d_patt, m, dout, nullptr, dim_out, 1))) return rc;
    if (ptr_kind == GGR_PTR_HOST) {
        CUDA_TRY(c, cudaMemcpyAsync(xb2, dout, (size_t)m * dim_out * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        return take_device_error(c, "a bounded wait inside a kernel ran out");
    }
    return GGR_OK;
}
