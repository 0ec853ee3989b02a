/*
 * TEST INFRASTRUCTURE - CPU oracle (see ref_attention.h). Each function names
 * the reference lines it restates (paths inside apimeister/gguf-runner).
 * x86 / scalar branches only; the reference's NEON branches use a polynomial
 * exp and round-to-even and are not what an x86 host runs.
 *
 * Build with strict IEEE semantics (-O2 -ffp-contract=off, no fast-math) so
 * summation order and rounding equal the reference's scalar Rust loops.
 */
#include "ref_attention.h"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

namespace {

// src/engine/io/gguf.rs:107-116 (round to nearest even, NaN keeps a payload)
inline uint16_t f32_to_bf16(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 64);
    return (uint16_t)((bits + (0x7fffu + ((bits >> 16) & 1u))) >> 16);
}
// src/engine/io/gguf.rs:54-57
inline float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

struct Block {
    int64_t start, len;
};

}  // namespace

// Persistent worker pool standing in for the reference's rayon fan-out over
// query heads (src/engine/runtime/inference.rs:2002-2007). Each head is still
// computed by one thread in a fixed order, so the thread count never changes
// a result.
class HeadPool {
public:
    explicit HeadPool(int n) : n_(n) {
        for (int i = 1; i < n_; ++i) workers_.emplace_back([this, i] { loop(i); });
    }
    ~HeadPool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
            ++gen_;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    int size() const { return n_; }
    void run(int count, const std::function<void(int)>& fn) {
        if (n_ == 1 || count <= 1) {
            for (int i = 0; i < count; ++i) fn(i);
            return;
        }
        {
            std::lock_guard<std::mutex> g(m_);
            fn_ = &fn;
            count_ = count;
            next_.store(0);
            pending_ = n_ - 1;
            ++gen_;
        }
        cv_.notify_all();
        work();
        std::unique_lock<std::mutex> g(m_);
        done_.wait(g, [this] { return pending_ == 0; });
    }

private:
    void work() {
        for (;;) {
            int i = next_.fetch_add(1);
            if (i >= count_) break;
            (*fn_)(i);
        }
    }
    void loop(int) {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
            }
            work();
            {
                std::lock_guard<std::mutex> g(m_);
                if (--pending_ == 0) done_.notify_one();
            }
        }
    }
    int n_;
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    const std::function<void(int)>* fn_ = nullptr;
    int count_ = 0, pending_ = 0;
    std::atomic<int> next_{0};
    uint64_t gen_ = 0;
    bool stop_ = false;
};

struct ora_plan {
    std::vector<std::array<int64_t, 3>> positions;
    int64_t next_text = 0;
};

struct ora_ctx {
    ora_config c;
    std::vector<int32_t> windows;
    int D, kv_dim, q_dim, G, rope_half;
    float attn_scale;
    std::vector<float> freqs, freqs_swa;
    int threads = 1;
    HeadPool* pool = nullptr;
    // storage (one of)
    std::vector<float> kf, vf;
    std::vector<uint16_t> kh, vh;
    std::vector<int8_t> kq, vq;
    std::vector<float> ks, vs;
    // TurboQuant storage (kv_format 4): 2-bit codes, residual sign bits, sigma (ks / vs) and residual norm per
    // (row, kv head), and the sign tables of the four transforms
    std::vector<uint8_t> kt_base, vt_base, kt_sign, vt_sign, turbo_signs;
    std::vector<float> k_rnorm, v_rnorm;
    // plans
    bool has_plan = false;
    ora_plan plan;
    std::vector<Block> blocks;
    int64_t prompt_tokens = 0;
    // per-layer fixups (empty = absent)
    std::vector<std::vector<float>> q_bias, k_bias, v_bias, q_norm, k_norm;
    float norm_eps = 1e-6f;
    // scratch: att rows per head (src/engine/runtime/inference.rs:1611-1614)
    std::vector<float> att;
};

namespace {

// src/engine/positions.rs:46-54
inline void plan_at(const ora_plan& p, int64_t pos, int64_t out[3]) {
    if (pos >= 0 && (size_t)pos < p.positions.size()) {
        out[0] = p.positions[pos][0];
        out[1] = p.positions[pos][1];
        out[2] = p.positions[pos][2];
    } else {
        int64_t v = p.next_text + (pos - (int64_t)p.positions.size());
        out[0] = out[1] = out[2] = v;
    }
}

// src/engine/positions.rs:57-72
inline int rope_axis(int layout, int frequency, const int32_t sections[4]) {
    if (layout == 0) return 0;
    int axis = frequency % 3;
    if (axis != 0 && frequency / 3 < sections[axis]) return axis;
    return 0;
}

// src/engine/runtime/inference.rs:1821-1825
inline bool is_swa_layer(const ora_ctx* s, int l) {
    if (s->windows.empty()) return s->c.swa_pattern > 0 && (l % s->c.swa_pattern < s->c.swa_pattern - 1);
    return s->windows[l] != 0;
}

// src/engine/runtime/inference.rs:1485-1523
void rope_angles(const ora_ctx* s, int l, int64_t pos, float* cs, float* sn) {
    bool swa = is_swa_layer(s, l);
    const std::vector<float>& fr = (s->c.swa_theta_on_window_layers && swa) ? s->freqs_swa : s->freqs;
    int64_t coord[3] = {pos, pos, pos};
    if (s->has_plan) plan_at(s->plan, pos, coord);
    float fscale = swa ? s->c.rope_scale_local : s->c.rope_scale_global;
    for (int i = 0; i < s->rope_half; ++i) {
        int axis = rope_axis(s->c.rope_layout, i, s->c.rope_sections);
        float val = ((float)coord[axis] * fr[i]) * fscale;
        cs[i] = cosf(val);
        sn[i] = sinf(val);
    }
}

// src/engine/runtime/inference.rs:1817-1874
void apply_rope(const ora_ctx* s, int l, int64_t pos, float* q, float* k) {
    std::vector<float> cs(s->rope_half), sn(s->rope_half);
    rope_angles(s, l, pos, cs.data(), sn.data());
    const int D = s->D, half = s->rope_half;
    if (s->c.rope_style == 0) {
        for (int pass = 0; pass < 2; ++pass) {
            float* x = pass == 0 ? q : k;
            int nh = pass == 0 ? s->c.n_heads : s->c.n_kv_heads;
            for (int h = 0; h < nh; ++h) {
                float* p = x + (size_t)h * D;
                for (int i = 0; i < half; ++i) {
                    float c = cs[i], sgn = sn[i];
                    float v0 = p[i], v1 = p[i + half];
                    p[i] = v0 * c - v1 * sgn;
                    p[i + half] = v0 * sgn + v1 * c;
                }
            }
        }
    } else {
        for (int i = 0; i < s->q_dim; i += 2) {
            int idx = (i % D) / 2;
            float c = cs[idx], sgn = sn[idx];
            int rotn = i < s->kv_dim ? 2 : 1;
            for (int v = 0; v < rotn; ++v) {
                float* x = v == 0 ? q : k;
                float v0 = x[i], v1 = x[i + 1];
                x[i] = v0 * c - v1 * sgn;
                x[i + 1] = v0 * sgn + v1 * c;
            }
        }
    }
    if (s->c.scale_mode == 1) {
        for (int i = 0; i < s->q_dim; ++i) q[i] *= s->attn_scale;
    }
}

// src/engine/runtime/inference.rs:251-267 (non-aarch64 branch)
void quantize_row_q8(const float* src, int n, int8_t* dst, float* scale_out) {
    float max_abs = 0.0f;
    for (int i = 0; i < n; ++i) max_abs = std::max(max_abs, std::fabs(src[i]));
    if (max_abs == 0.0f) {
        *scale_out = 1.0f;
        std::memset(dst, 0, n);
        return;
    }
    float inv = 127.0f / max_abs;
    *scale_out = max_abs / 127.0f;
    for (int i = 0; i < n; ++i) {
        float r = roundf(src[i] * inv);
        r = std::min(127.0f, std::max(-127.0f, r));
        dst[i] = (int8_t)r;
    }
}

inline size_t row_index(const ora_ctx* s, int seq, int l, int64_t pos) {
    return ((size_t)seq * s->c.n_layers + l) * (size_t)s->c.seq_len + (size_t)pos;
}

// ---- TurboQuant cache format (src/engine/runtime/inference.rs:349-1334, scalar branches) ----------------

const float kTurboCentroids[4] = {-1.510417f, -0.45278f, 0.45278f, 1.510417f};  // :349
const float kTurboThreshold = 0.9815985f;                                       // :350-351
const uint64_t kTurboSalts[4] = {0x9E3779B97F4A7C15ull, 0xC2B2AE3D27D4EB4Full, 0x165667B19E3779F9ull,
                                 0xD6E8FEB86659FD93ull};  // rot_pre, rot_post, res_pre, res_post (:352-355)

// :673-679
inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline int turbo_sign_bytes(int D) { return (D + 7) / 8; }

// :370-395: bit = 1 means multiply by -1; layout [slot][layer][kv_head][bytes]
void turbo_build_sign_table(ora_ctx* s) {
    const int L = s->c.n_layers, H = s->c.n_kv_heads, D = s->D, bytes = turbo_sign_bytes(D);
    s->turbo_signs.assign((size_t)4 * L * H * bytes, 0);
    const size_t stride = (size_t)L * H * bytes;
    for (int slot = 0; slot < 4; ++slot)
        for (int l = 0; l < L; ++l)
            for (int h = 0; h < H; ++h) {
                uint64_t seed = splitmix64(((uint64_t)l << 32) ^ (uint64_t)h ^ kTurboSalts[slot]);
                uint8_t* bits = &s->turbo_signs[slot * stride + ((size_t)l * H + h) * bytes];
                for (int i = 0; i < D; ++i)
                    if (splitmix64(seed ^ (uint64_t)i) & 1) bits[i / 8] |= (uint8_t)(1u << (i & 7));
            }
}

inline const uint8_t* turbo_sign_slot(const ora_ctx* s, int slot, int l, int kvh) {
    const int bytes = turbo_sign_bytes(s->D);
    const size_t stride = (size_t)s->c.n_layers * s->c.n_kv_heads * bytes;
    return &s->turbo_signs[slot * stride + ((size_t)l * s->c.n_kv_heads + kvh) * bytes];
}

// :441-456 scalar tail
inline void turbo_apply_signs(float* v, int n, const uint8_t* bits) {
    for (int i = 0; i < n; ++i)
        if ((bits[i / 8] >> (i & 7)) & 1) v[i] = -v[i];
}

// :681-701 and :822-833: skipped when n is not a power of two
inline void turbo_fwht(float* v, int n) {
    if (n <= 0 || (n & (n - 1)) != 0) return;
    for (int width = 1; width < n; width *= 2)
        for (int base = 0; base < n; base += 2 * width)
            for (int i = 0; i < width; ++i) {
                float a = v[base + i], b = v[base + i + width];
                v[base + i] = a + b;
                v[base + i + width] = a - b;
            }
    float scale = 1.0f / sqrtf((float)n);
    for (int i = 0; i < n; ++i) v[i] *= scale;
}

// :595-605
inline void turbo_transform(float* v, int n, const uint8_t* first, const uint8_t* second) {
    turbo_apply_signs(v, n, first);
    turbo_fwht(v, n);
    turbo_apply_signs(v, n, second);
}

// src/engine/kernels/math.rs:467-473
inline float l2_norm(const float* x, int n) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    return sqrtf(ss);
}

// :835-845
inline int turbo_code(float x) {
    if (x < -kTurboThreshold) return 0;
    if (x < 0.0f) return 1;
    if (x < kTurboThreshold) return 2;
    return 3;
}

inline int get_q2(const uint8_t* src, size_t e) { return (src[e / 4] >> ((e & 3) * 2)) & 3; }
inline void set_q2(uint8_t* dst, size_t e, int code) {
    const int sh = (int)(e & 3) * 2;
    dst[e / 4] = (uint8_t)((dst[e / 4] & ~(3u << sh)) | ((unsigned)code << sh));
}
inline bool get_bit(const uint8_t* src, size_t e) { return (src[e / 8] >> (e & 7)) & 1; }
inline void set_bit(uint8_t* dst, size_t e, bool on) {
    if (on) dst[e / 8] |= (uint8_t)(1u << (e & 7));
    else dst[e / 8] &= (uint8_t)~(1u << (e & 7));
}

// :885-952: one head of one row
void turbo_quantize_head(const ora_ctx* s, const float* src, int l, int kvh, uint8_t* base, uint8_t* sign,
                         size_t elem_offset, float* scale_out, float* rnorm_out) {
    const int D = s->D;
    std::vector<float> rot(src, src + D), res(D);
    turbo_transform(rot.data(), D, turbo_sign_slot(s, 0, l, kvh), turbo_sign_slot(s, 1, l, kvh));
    float sigma = l2_norm(rot.data(), D) / sqrtf((float)D);
    *scale_out = sigma;
    if (sigma == 0.0f) {
        *rnorm_out = 0.0f;
        for (int i = 0; i < D; ++i) {
            set_q2(base, elem_offset + i, 0);
            set_bit(sign, elem_offset + i, true);
        }
        return;
    }
    float inv_sigma = 1.0f / sigma;
    for (int i = 0; i < D; ++i) {
        int code = turbo_code(rot[i] * inv_sigma);
        res[i] = rot[i] - kTurboCentroids[code] * sigma;
        set_q2(base, elem_offset + i, code);
    }
    float gamma = l2_norm(res.data(), D);
    *rnorm_out = gamma;
    if (gamma == 0.0f) {
        for (int i = 0; i < D; ++i) set_bit(sign, elem_offset + i, true);
        return;
    }
    for (int i = 0; i < D; ++i) res[i] /= gamma;
    turbo_transform(res.data(), D, turbo_sign_slot(s, 2, l, kvh), turbo_sign_slot(s, 3, l, kvh));
    for (int i = 0; i < D; ++i) set_bit(sign, elem_offset + i, res[i] >= 0.0f);
}

// :975-982
inline float turbo_residual_scale(int D, float rnorm) {
    if (rnorm == 0.0f) return 0.0f;
    return rnorm * sqrtf(1.57079632679489661923f / (float)D);
}

// :1246-1269
inline float turbo_dot(const ora_ctx* s, const float* qr, const float* qp, const uint8_t* base, const uint8_t* sign,
                       size_t off, float scale, float rnorm) {
    const int D = s->D;
    float acc = 0.0f;
    if (scale != 0.0f)
        for (int i = 0; i < D; ++i) acc += qr[i] * (kTurboCentroids[get_q2(base, off + i)] * scale);
    float rs = turbo_residual_scale(D, rnorm);
    if (rs != 0.0f)
        for (int i = 0; i < D; ++i) acc += get_bit(sign, off + i) ? rs * qp[i] : -rs * qp[i];
    return acc;
}

// :1284-1306
inline void turbo_axpy(const ora_ctx* s, float* base_acc, float* res_acc, float a, const uint8_t* base,
                       const uint8_t* sign, size_t off, float scale, float rnorm) {
    const int D = s->D;
    if (scale != 0.0f)
        for (int i = 0; i < D; ++i) base_acc[i] += a * kTurboCentroids[get_q2(base, off + i)] * scale;
    float rs = a * turbo_residual_scale(D, rnorm);
    if (rs != 0.0f)
        for (int i = 0; i < D; ++i) res_acc[i] += get_bit(sign, off + i) ? rs : -rs;
}

// src/engine/runtime/inference.rs:1877-1918
void kv_write(ora_ctx* s, int seq, int l, int64_t pos, const float* k, const float* v) {
    size_t r = row_index(s, seq, l, pos);
    size_t off = r * s->kv_dim;
    switch (s->c.kv_format) {
        case 0:
            std::memcpy(&s->kf[off], k, sizeof(float) * s->kv_dim);
            std::memcpy(&s->vf[off], v, sizeof(float) * s->kv_dim);
            break;
        case 1:
            for (int i = 0; i < s->kv_dim; ++i) {
                s->kh[off + i] = f32_to_bf16(k[i]);
                s->vh[off + i] = f32_to_bf16(v[i]);
            }
            break;
        case 2:
            quantize_row_q8(k, s->kv_dim, &s->kq[off], &s->ks[r]);
            quantize_row_q8(v, s->kv_dim, &s->vq[off], &s->vs[r]);
            break;
        case 3: {
            int nb = s->kv_dim / 32;
            for (int b = 0; b < nb; ++b) {
                quantize_row_q8(k + b * 32, 32, &s->kq[off + b * 32], &s->ks[r * nb + b]);
                quantize_row_q8(v + b * 32, 32, &s->vq[off + b * 32], &s->vs[r * nb + b]);
            }
            break;
        }
        case 4:  // :1919-1963
            for (int h = 0; h < s->c.n_kv_heads; ++h) {
                size_t aux = r * s->c.n_kv_heads + h, eo = off + (size_t)h * s->D;
                turbo_quantize_head(s, k + (size_t)h * s->D, l, h, s->kt_base.data(), s->kt_sign.data(), eo, &s->ks[aux],
                                    &s->k_rnorm[aux]);
                turbo_quantize_head(s, v + (size_t)h * s->D, l, h, s->vt_base.data(), s->vt_sign.data(), eo, &s->vs[aux],
                                    &s->v_rnorm[aux]);
            }
            break;
    }
}

// src/engine/runtime/attention.rs:30-39
const Block* block_at(const ora_ctx* s, int64_t position) {
    size_t idx = 0;
    while (idx < s->blocks.size() && s->blocks[idx].start <= position) ++idx;
    if (idx == 0) return nullptr;
    const Block& b = s->blocks[idx - 1];
    if (position - b.start < b.len) return &b;
    return nullptr;
}

// src/engine/runtime/attention.rs:73-97
void visible_keys(const ora_ctx* s, int l, int64_t query, int64_t* start, int64_t* end) {
    int64_t e = query + 1;
    int64_t st = 0;
    if (!s->windows.empty() && l < (int)s->windows.size() && s->windows[l] != 0)
        st = std::max<int64_t>(0, e - s->windows[l]);
    if (s->c.image_mode == 1) {
        const Block* b = block_at(s, query);
        if (b) {
            *start = std::min(st, b->start);
            *end = b->start + b->len;
            return;
        }
    }
    *start = st;
    *end = e;
}

// src/engine/runtime/inference.rs:1343-1349 and :1360-1365 (q8), same loops on
// exact / bf16-rounded values for the f32 and bf16 stores.
struct RowReader {
    const ora_ctx* s;
    int fmt;
    inline float dot(const float* q, size_t r, int kvh) const {
        const int D = s->D;
        size_t off = r * s->kv_dim + (size_t)kvh * D;
        float acc = 0.0f;
        switch (fmt) {
            case 0:
                for (int i = 0; i < D; ++i) acc += q[i] * s->kf[off + i];
                break;
            case 1:
                for (int i = 0; i < D; ++i) acc += q[i] * bf16_to_f32(s->kh[off + i]);
                break;
            case 2: {
                float sc = s->ks[r];
                for (int i = 0; i < D; ++i) acc += q[i] * ((float)s->kq[off + i] * sc);
                break;
            }
            case 3: {
                // src/engine/runtime/inference.rs:1369-1418: per-block partial sums
                int nbh = D / 32, nb = s->kv_dim / 32;
                const float* sc = &s->ks[r * nb + (size_t)kvh * nbh];
                for (int b = 0; b < nbh; ++b) {
                    float part = 0.0f;
                    for (int i = 0; i < 32; ++i)
                        part += q[b * 32 + i] * ((float)s->kq[off + b * 32 + i] * sc[b]);
                    acc += part;
                }
                break;
            }
        }
        return acc;
    }
    inline void axpy(float* dst, float a, size_t r, int kvh) const {
        const int D = s->D;
        size_t off = r * s->kv_dim + (size_t)kvh * D;
        switch (fmt) {
            case 0:
                for (int i = 0; i < D; ++i) dst[i] += a * s->vf[off + i];
                break;
            case 1:
                for (int i = 0; i < D; ++i) dst[i] += a * bf16_to_f32(s->vh[off + i]);
                break;
            case 2: {
                float scaled = a * s->vs[r];
                for (int i = 0; i < D; ++i) dst[i] += scaled * (float)s->vq[off + i];
                break;
            }
            case 3: {
                int nbh = D / 32, nb = s->kv_dim / 32;
                const float* sc = &s->vs[r * nb + (size_t)kvh * nbh];
                for (int b = 0; b < nbh; ++b) {
                    float scaled = a * sc[b];
                    for (int i = 0; i < 32; ++i) dst[b * 32 + i] += scaled * (float)s->vq[off + b * 32 + i];
                }
                break;
            }
        }
    }
};

// src/engine/kernels/math.rs:263-280 (scalar branch)
void softmax_scalar(float* x, int64_t size) {
    float max_val = x[0];
    for (int64_t i = 1; i < size; ++i)
        if (x[i] > max_val) max_val = x[i];
    float sum = 0.0f;
    for (int64_t i = 0; i < size; ++i) {
        x[i] = expf(x[i] - max_val);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (int64_t i = 0; i < size; ++i) x[i] *= inv;
}

// The TurboQuant arm of attention_token (src/engine/runtime/inference.rs:2301-2527): the query is rotated and
// projected once per head (:954-968), scores and value sums read the packed codes, and the two accumulators go
// through the inverse transforms at the end (:1323-1334).
void attention_head_turbo(ora_ctx* s, int seq, int l, int h, int64_t vs, int64_t ve, const float* q, float* out,
                          float* att) {
    const int D = s->D, Hkv = s->c.n_kv_heads;
    const int kvh = h / s->G;
    float* xb = out + (size_t)h * D;
    const uint8_t* rot_pre = turbo_sign_slot(s, 0, l, kvh);
    const uint8_t* rot_post = turbo_sign_slot(s, 1, l, kvh);
    const uint8_t* res_pre = turbo_sign_slot(s, 2, l, kvh);
    const uint8_t* res_post = turbo_sign_slot(s, 3, l, kvh);
    std::vector<float> qr(q + (size_t)h * D, q + (size_t)(h + 1) * D), qp, res(D, 0.0f);
    turbo_transform(qr.data(), D, rot_pre, rot_post);
    qp = qr;
    turbo_transform(qp.data(), D, res_pre, res_post);
    const bool apply_scale = s->c.scale_mode == 0;
    const size_t base = row_index(s, seq, l, 0);
    auto score_at = [&](int64_t t) {
        size_t r = base + t, aux = r * Hkv + kvh, off = r * s->kv_dim + (size_t)kvh * D;
        float sc = turbo_dot(s, qr.data(), qp.data(), s->kt_base.data(), s->kt_sign.data(), off, s->ks[aux], s->k_rnorm[aux]);
        if (apply_scale) sc *= s->attn_scale;
        return sc;
    };
    auto value_at = [&](int64_t t, float a) {
        size_t r = base + t, aux = r * Hkv + kvh, off = r * s->kv_dim + (size_t)kvh * D;
        turbo_axpy(s, xb, res.data(), a, s->vt_base.data(), s->vt_sign.data(), off, s->vs[aux], s->v_rnorm[aux]);
    };
    for (int i = 0; i < D; ++i) xb[i] = 0.0f;
    if (s->c.softmax_mode == 1) {
        float max_score = -std::numeric_limits<float>::infinity(), score_sum = 0.0f;
        for (int64_t t = vs; t < ve; ++t) {
            float score = score_at(t);
            if (score > max_score) {
                if (score_sum > 0.0f) {
                    float rescale = expf(max_score - score);
                    for (int i = 0; i < D; ++i) {
                        xb[i] *= rescale;
                        res[i] *= rescale;
                    }
                    score_sum *= rescale;
                }
                max_score = score;
            }
            float w = expf(score - max_score);
            score_sum += w;
            value_at(t, w);
        }
        if (score_sum > 0.0f) {
            float inv = 1.0f / score_sum;
            for (int i = 0; i < D; ++i) {
                xb[i] *= inv;
                res[i] *= inv;
            }
        }
    } else {
        int64_t n = ve - vs;
        for (int64_t t = 0; t < n; ++t) att[t] = score_at(vs + t);
        softmax_scalar(att, n);
        for (int64_t t = 0; t < n; ++t) value_at(vs + t, att[t]);
    }
    // :1323-1334
    turbo_transform(res.data(), D, res_post, res_pre);
    for (int i = 0; i < D; ++i) xb[i] += res[i];
    turbo_transform(xb, D, rot_post, rot_pre);
}

// src/engine/runtime/inference.rs:2286-2529 (serial branch; the rayon branch
// :2002-2283 does the same arithmetic per head on worker threads)
void attention_head(ora_ctx* s, int seq, int l, int h, int64_t vs, int64_t ve, const float* q, float* out,
                    float* att) {
    if (s->c.kv_format == 4) {
        attention_head_turbo(s, seq, l, h, vs, ve, q, out, att);
        return;
    }
    const int D = s->D;
    const float* qh = q + (size_t)h * D;
    int kvh = h / s->G;
    float* xb = out + (size_t)h * D;
    RowReader rd{s, s->c.kv_format};
    bool apply_scale = s->c.scale_mode == 0;
    size_t base = row_index(s, seq, l, 0);
    if (s->c.softmax_mode == 1) {
        // :2320-2429 online variant
        for (int i = 0; i < D; ++i) xb[i] = 0.0f;
        float max_score = -std::numeric_limits<float>::infinity();
        float score_sum = 0.0f;
        for (int64_t t = vs; t < ve; ++t) {
            float score = rd.dot(qh, base + t, kvh);
            if (apply_scale) score *= s->attn_scale;
            if (score > max_score) {
                if (score_sum > 0.0f) {
                    float rescale = expf(max_score - score);
                    for (int i = 0; i < D; ++i) xb[i] *= rescale;
                    score_sum *= rescale;
                }
                max_score = score;
            }
            float w = expf(score - max_score);
            score_sum += w;
            rd.axpy(xb, w, base + t, kvh);
        }
        if (score_sum > 0.0f) {
            float inv = 1.0f / score_sum;
            for (int i = 0; i < D; ++i) xb[i] *= inv;
        }
    } else {
        // :2430-2527 two-pass variant
        int64_t n = ve - vs;
        for (int64_t t = 0; t < n; ++t) {
            float score = rd.dot(qh, base + vs + t, kvh);
            if (apply_scale) score *= s->attn_scale;
            att[t] = score;
        }
        softmax_scalar(att, n);
        for (int i = 0; i < D; ++i) xb[i] = 0.0f;
        for (int64_t t = 0; t < n; ++t) rd.axpy(xb, att[t], base + vs + t, kvh);
    }
}

// src/engine/kernels/math.rs:164-184
void rmsnorm_per_head(float* x, const float* weight, int n_heads, int head_size, float eps) {
    for (int h = 0; h < n_heads; ++h) {
        float* p = x + (size_t)h * head_size;
        float ss = 0.0f;
        for (int j = 0; j < head_size; ++j) ss += p[j] * p[j];
        ss /= (float)head_size;
        ss += eps;
        ss = 1.0f / sqrtf(ss);
        for (int j = 0; j < head_size; ++j) p[j] = weight[j] * (ss * p[j]);
    }
}

// src/engine/runtime/inference.rs:2535-2572
void qkv_bias_and_norm(const ora_ctx* s, int l, float* q, float* k, float* v) {
    if ((size_t)l < s->q_bias.size() && !s->q_bias[l].empty()) {
        for (int i = 0; i < s->q_dim; ++i) q[i] += s->q_bias[l][i];
        for (int i = 0; i < s->kv_dim; ++i) {
            k[i] += s->k_bias[l][i];
            v[i] += s->v_bias[l][i];
        }
    }
    if ((size_t)l < s->q_norm.size() && !s->q_norm[l].empty() && !s->k_norm[l].empty()) {
        const float eps = s->norm_eps > 0.0f ? s->norm_eps : 1e-5f;
        rmsnorm_per_head(q, s->q_norm[l].data(), s->c.n_heads, s->D, eps);
        rmsnorm_per_head(k, s->k_norm[l].data(), s->c.n_kv_heads, s->D, eps);
    }
}

void attention_token(ora_ctx* s, int seq, int l, int64_t pos, const float* q, float* out) {
    int64_t vs, ve;
    visible_keys(s, l, pos, &vs, &ve);
    const int H = s->c.n_heads;
    const size_t S = (size_t)s->c.seq_len;
    if ((size_t)s->att.size() < (size_t)H * S) s->att.resize((size_t)H * S);
    float* att = s->att.data();
    if (s->pool && s->threads > 1) {
        s->pool->run(H, [&](int h) { attention_head(s, seq, l, h, vs, ve, q, out, att + (size_t)h * S); });
    } else {
        for (int h = 0; h < H; ++h) attention_head(s, seq, l, h, vs, ve, q, out, att + (size_t)h * S);
    }
}

}  // namespace

extern "C" {

// src/engine/runtime/inference.rs:1529-1748 (KV and RoPE parts only)
int ora_create(const ora_config* cfg, ora_ctx** out, const char** err) {
    static const char* e_scale = "RoPE frequency scales must be finite and positive";
    static const char* e_win = "attention policy requires one positive window or global entry per layer";
    static const char* e_shape = "invalid attention shape";
    const char* dummy;
    if (!err) err = &dummy;
    *err = nullptr;
    float sc[2] = {cfg->rope_scale_global, cfg->rope_scale_local};
    for (float v : sc)
        if (!std::isfinite(v) || v <= 0.0f) {
            *err = e_scale;
            return -1;
        }
    if (cfg->n_layer_windows != 0) {
        bool bad = cfg->n_layer_windows != cfg->n_layers;
        for (int i = 0; !bad && i < cfg->n_layer_windows; ++i) bad = cfg->layer_windows[i] < 0;
        if (bad) {
            *err = e_win;
            return -2;
        }
    }
    if (cfg->n_layers <= 0 || cfg->n_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->head_dim <= 0 ||
        cfg->n_heads % cfg->n_kv_heads != 0 || cfg->seq_len <= 0 || cfg->max_batch <= 0) {
        *err = e_shape;
        return -3;
    }
    ora_ctx* s = new ora_ctx();
    s->c = *cfg;
    s->windows.assign(cfg->layer_windows, cfg->layer_windows + cfg->n_layer_windows);
    s->c.layer_windows = nullptr;
    s->D = cfg->head_dim;
    s->kv_dim = cfg->n_kv_heads * s->D;
    s->q_dim = cfg->n_heads * s->D;
    s->G = cfg->n_heads / cfg->n_kv_heads;
    int rope_dim = cfg->rope_dim > 0 ? cfg->rope_dim : s->D;  // :1590-1594
    s->c.rope_dim = rope_dim;
    s->rope_half = rope_dim / 2;
    s->freqs.resize(s->rope_half);
    s->freqs_swa.resize(s->rope_half);
    float swa_theta = cfg->rope_theta_swa > 0.0f ? cfg->rope_theta_swa : 10000.0f;  // :1601-1605
    for (int i = 0; i < s->rope_half; ++i) {
        float e = (float)(i * 2) / (float)rope_dim;
        s->freqs[i] = 1.0f / powf(cfg->rope_theta, e);  // :1596-1599
        s->freqs_swa[i] = 1.0f / powf(swa_theta, e);     // :1606-1609
    }
    s->attn_scale = 1.0f / sqrtf((float)s->D);  // :1745
    size_t rows = (size_t)cfg->max_batch * cfg->n_layers * cfg->seq_len;
    size_t elems = rows * s->kv_dim;
    switch (cfg->kv_format) {
        case 0:
            s->kf.assign(elems, 0.0f);
            s->vf.assign(elems, 0.0f);
            break;
        case 1:
            s->kh.assign(elems, 0);
            s->vh.assign(elems, 0);
            break;
        case 2:
            s->kq.assign(elems, 0);
            s->vq.assign(elems, 0);
            s->ks.assign(rows, 0.0f);
            s->vs.assign(rows, 0.0f);
            break;
        case 3:
            s->kq.assign(elems, 0);
            s->vq.assign(elems, 0);
            s->ks.assign(rows * (size_t)std::max(1, s->kv_dim / 32), 0.0f);
            s->vs.assign(rows * (size_t)std::max(1, s->kv_dim / 32), 0.0f);
            break;
        case 4: {
            size_t aux = rows * (size_t)cfg->n_kv_heads;
            s->kt_base.assign((elems + 3) / 4, 0);
            s->vt_base.assign((elems + 3) / 4, 0);
            s->kt_sign.assign((elems + 7) / 8, 0);
            s->vt_sign.assign((elems + 7) / 8, 0);
            s->ks.assign(aux, 0.0f);
            s->vs.assign(aux, 0.0f);
            s->k_rnorm.assign(aux, 0.0f);
            s->v_rnorm.assign(aux, 0.0f);
            turbo_build_sign_table(s);
            break;
        }
        default:
            delete s;
            *err = e_shape;
            return -3;
    }
    *out = s;
    return 0;
}

void ora_destroy(ora_ctx* ctx) {
    if (!ctx) return;
    delete ctx->pool;
    delete ctx;
}

void ora_set_threads(ora_ctx* ctx, int n) {
    n = n < 1 ? 1 : n;
    if (ctx->pool && ctx->pool->size() != n) {
        delete ctx->pool;
        ctx->pool = nullptr;
    }
    if (n > 1 && !ctx->pool) ctx->pool = new HeadPool(n);
    ctx->threads = n;
}

int ora_threads_available(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : (int)n;
}

int ora_set_position_plan(ora_ctx* ctx, const int32_t* thw, int32_t n, int32_t next_text_pos) {
    ctx->plan.positions.clear();
    for (int i = 0; i < n; ++i) ctx->plan.positions.push_back({thw[3 * i], thw[3 * i + 1], thw[3 * i + 2]});
    ctx->plan.next_text = next_text_pos;
    ctx->has_plan = n > 0 || next_text_pos != 0;
    return 0;
}

// src/engine/runtime/attention.rs:9-28
int ora_media_plan_validate(const int64_t* sl, int32_t n, int64_t prompt_tokens) {
    int64_t previous_end = 0;
    for (int i = 0; i < n; ++i) {
        int64_t st = sl[2 * i], len = sl[2 * i + 1];
        if (st < 0 || len < 0) return -1;
        if (len > std::numeric_limits<int64_t>::max() - st) return -1;
        int64_t end = st + len;
        if (len == 0 || st < previous_end || end > prompt_tokens) return -1;
        previous_end = end;
    }
    return 0;
}

int ora_set_media_blocks(ora_ctx* ctx, const int32_t* start_len, int32_t n, int32_t prompt_tokens) {
    std::vector<int64_t> sl(2 * (size_t)n);
    for (int i = 0; i < 2 * n; ++i) sl[i] = start_len[i];
    if (ora_media_plan_validate(sl.data(), n, prompt_tokens) != 0) return -1;
    ctx->blocks.clear();
    for (int i = 0; i < n; ++i) ctx->blocks.push_back({sl[2 * i], sl[2 * i + 1]});
    ctx->prompt_tokens = prompt_tokens;
    return 0;
}

// src/engine/runtime/attention.rs:43-70
int64_t ora_media_chunk_end(const int64_t* sl, int32_t n, int64_t prompt_tokens, int64_t start, int64_t limit,
                            int64_t chunk) {
    if (chunk == 0 || start >= limit || limit > prompt_tokens) return -1;
    // block_at(start)
    int idx = 0;
    while (idx < n && sl[2 * idx] <= start) ++idx;
    if (idx > 0 && start - sl[2 * (idx - 1)] < sl[2 * (idx - 1) + 1]) {
        int64_t bs = sl[2 * (idx - 1)], bl = sl[2 * (idx - 1) + 1];
        if (start != bs) return -2;
        int64_t end = bs + bl;
        if (end > limit) return -3;
        return end;
    }
    int64_t end = (chunk > std::numeric_limits<int64_t>::max() - start) ? std::numeric_limits<int64_t>::max()
                                                                         : start + chunk;
    end = std::min(end, limit);
    for (int i = 0; i < n; ++i)
        if (sl[2 * i] >= start && sl[2 * i] < end) return sl[2 * i];
    return end;
}

int ora_set_layer_fixups(ora_ctx* s, int32_t layer, const float* q_bias, const float* k_bias, const float* v_bias,
                         const float* q_norm, const float* k_norm, float eps) {
    if (layer < 0 || layer >= s->c.n_layers) return -1;
    const size_t L = (size_t)s->c.n_layers;
    for (auto* vec : {&s->q_bias, &s->k_bias, &s->v_bias, &s->q_norm, &s->k_norm}) vec->resize(L);
    s->q_bias[layer].clear();
    s->k_bias[layer].clear();
    s->v_bias[layer].clear();
    s->q_norm[layer].clear();
    s->k_norm[layer].clear();
    if (q_bias && k_bias && v_bias) {
        s->q_bias[layer].assign(q_bias, q_bias + s->q_dim);
        s->k_bias[layer].assign(k_bias, k_bias + s->kv_dim);
        s->v_bias[layer].assign(v_bias, v_bias + s->kv_dim);
    }
    if (q_norm && k_norm) {
        s->q_norm[layer].assign(q_norm, q_norm + s->D);
        s->k_norm[layer].assign(k_norm, k_norm + s->D);
    }
    s->norm_eps = eps;
    return 0;
}
void ora_qkv_bias_and_norm(ora_ctx* ctx, int32_t layer, float* q, float* k, float* v) {
    qkv_bias_and_norm(ctx, layer, q, k, v);
}

// Output gate of the decode call site (src/engine/runtime/inference.rs:3509-3519): per head
// sigmoid_mul_inplace (scalar branch, src/engine/kernels/math.rs:399-402: s = 1 / (1 + exp(-g)),
// d = finite_or_zero(d * s)), then sanitize_finite_inplace over the row (:458-462).
void ora_sigmoid_gate(ora_ctx* ctx, float* xb, const float* gate, int32_t gate_head_stride) {
    const int D = ctx->D;
    for (int h = 0; h < ctx->c.n_heads; ++h) {
        float* dst = xb + (size_t)h * D;
        const float* g = gate + (size_t)h * gate_head_stride;
        for (int i = 0; i < D; ++i) {
            const float s = 1.0f / (1.0f + std::exp(-g[i]));
            const float v = dst[i] * s;
            dst[i] = std::isfinite(v) ? v : 0.0f;
        }
    }
    for (int i = 0; i < ctx->q_dim; ++i)
        if (!std::isfinite(xb[i])) xb[i] = 0.0f;
}

// ---- projections either side of the path (scalar branches of the reference's matmul) ----------------
// IEEE half to single, as src/engine/io/gguf.rs:27-52 (subnormals normalised, infinities and NaNs kept).
static float fp16_to_fp32(uint16_t h) {
    const uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
    int32_t exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x03ffu;
    uint32_t bits;
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
            bits = sign | ((uint32_t)(exp + (127 - 15)) << 23) | (mant << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (mant << 13);
    } else {
        bits = sign | ((uint32_t)(exp + (127 - 15)) << 23) | (mant << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// xout[r] = dot(row r of W, x) for one activation row, W in the GGML row layouts the reference multiplies with
// (matmul_quantized_with_scratch, src/engine/kernels/quant.rs:7225): wtype 0 = F32 (vec_dot_f32 :1167),
// 1 = BF16 (vec_dot_bf16 scalar tail :1313-1316), 2 = Q8_0 (vec_dot_q8_0 scalar branch :2043-2059: per block of 32,
// the f32 dot of x with the int8 codes, times the block's f16 scale), 3 = Q4_K, 4 = Q6_K. Sequential f32 sums.
void ora_matmul(int32_t wtype, int32_t rows, int32_t cols, const void* w, const float* x, float* xout) {
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    for (int r = 0; r < rows; ++r) {
        float sum = 0.0f;
        if (wtype == 0) {
            const float* row = reinterpret_cast<const float*>(wb) + (size_t)r * cols;
            for (int i = 0; i < cols; ++i) sum += x[i] * row[i];
        } else if (wtype == 1) {
            const uint16_t* row = reinterpret_cast<const uint16_t*>(wb) + (size_t)r * cols;
            for (int i = 0; i < cols; ++i) {
                const uint32_t bits = (uint32_t)row[i] << 16;
                float wv;
                std::memcpy(&wv, &bits, 4);
                sum += x[i] * wv;
            }
        } else if (wtype == 3) {
            // Q4_K (vec_dot_q4_k, scalar branch of the x86 build, src/engine/kernels/quant.rs:3490-3521): super-blocks
            // of 256 = f16 d, f16 dmin, 12 bytes of packed 6-bit (scale, min) pairs (get_scale_min_k4 :118-126),
            // 128 bytes of nibbles; four groups of 64 elements, low nibbles then high nibbles
            const int nb = cols / 256;
            const uint8_t* row = wb + (size_t)r * nb * 144;
            for (int b = 0; b < nb; ++b) {
                const uint8_t* blk = row + (size_t)b * 144;
                const float d = fp16_to_fp32((uint16_t)(blk[0] | (blk[1] << 8)));
                const float dmin = fp16_to_fp32((uint16_t)(blk[2] | (blk[3] << 8)));
                const uint8_t* sc = blk + 4;
                const uint8_t* q = blk + 16;
                const float* xb = x + (size_t)b * 256;
                auto scale_min = [&](int j, int* s_out, int* m_out) {
                    if (j < 4) {
                        *s_out = sc[j] & 63;
                        *m_out = sc[j + 4] & 63;
                    } else {
                        *s_out = (sc[j + 4] & 0x0f) | ((sc[j - 4] >> 6) << 4);
                        *m_out = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
                    }
                };
                float block_sum = 0.0f;
                int is = 0;
                for (int j = 0; j < 256; j += 64) {
                    int sc1, m1, sc2, m2;
                    scale_min(is, &sc1, &m1);
                    scale_min(is + 1, &sc2, &m2);
                    const float d1 = d * (float)sc1, m1f = dmin * (float)m1;
                    const float d2 = d * (float)sc2, m2f = dmin * (float)m2;
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t qv = q[l];
                        const float w0 = d1 * (float)(qv & 0x0f) - m1f;
                        const float w1 = d2 * (float)(qv >> 4) - m2f;
                        block_sum += xb[j + l] * w0 + xb[j + 32 + l] * w1;
                    }
                    q += 32;
                    is += 2;
                }
                sum += block_sum;
            }
        } else if (wtype == 4) {
            // Q6_K (vec_dot_q6_k, scalar branch of the x86 build, src/engine/kernels/quant.rs:3654-3690): super-blocks of
            // 256 = 128 bytes of low nibbles, 64 bytes of high bit pairs, 16 int8 scales (one per 16 weights), f16 d
            const int nb = cols / 256;
            const uint8_t* row = wb + (size_t)r * nb * 210;
            for (int b = 0; b < nb; ++b) {
                const uint8_t* blk = row + (size_t)b * 210;
                const float d = fp16_to_fp32((uint16_t)(blk[208] | (blk[209] << 8)));
                const uint8_t* ql = blk;
                const uint8_t* qh = blk + 128;
                const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
                const float* xb = x + (size_t)b * 256;
                float block_sum = 0.0f;
                for (int n_outer = 0; n_outer < 256; n_outer += 128) {
                    for (int l = 0; l < 32; ++l) {
                        const int is = l / 16;
                        const int q1 = (int)(int8_t)((ql[l] & 0x0f) | ((qh[l] & 0x03) << 4)) - 32;
                        const int q2 = (int)(int8_t)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 0x03) << 4)) - 32;
                        const int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 0x03) << 4)) - 32;
                        const int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 0x03) << 4)) - 32;
                        const float s0 = d * (float)sc[is], s1 = d * (float)sc[is + 2];
                        const float s2 = d * (float)sc[is + 4], s3 = d * (float)sc[is + 6];
                        block_sum += xb[n_outer + l] * (s0 * (float)q1);
                        block_sum += xb[n_outer + 32 + l] * (s1 * (float)q2);
                        block_sum += xb[n_outer + 64 + l] * (s2 * (float)q3);
                        block_sum += xb[n_outer + 96 + l] * (s3 * (float)q4);
                    }
                    ql += 64;
                    qh += 32;
                    sc += 8;
                }
                sum += block_sum;
            }
        } else {
            const int nb = cols / 32;
            const uint8_t* row = wb + (size_t)r * nb * 34;
            for (int b = 0; b < nb; ++b) {
                const uint8_t* blk = row + (size_t)b * 34;
                const float d = fp16_to_fp32((uint16_t)(blk[0] | (blk[1] << 8)));
                float block_sum = 0.0f;
                for (int j = 0; j < 32; ++j) block_sum += x[b * 32 + j] * (float)(int8_t)blk[2 + j];
                sum += block_sum * d;
            }
        }
        xout[r] = sum;
    }
}

float ora_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }

void ora_rope_angles(ora_ctx* ctx, int32_t layer, int32_t pos, float* c, float* s) {
    rope_angles(ctx, layer, pos, c, s);
}
void ora_apply_rope_qk(ora_ctx* ctx, int32_t layer, int32_t pos, float* q, float* k) {
    apply_rope(ctx, layer, pos, q, k);
}
void ora_kv_write_token(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* k, const float* v) {
    kv_write(ctx, seq, layer, pos, k, v);
}
void ora_attention_token(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* q, float* out) {
    attention_token(ctx, seq, layer, pos, q, out);
}
void ora_visible_keys(ora_ctx* ctx, int32_t layer, int32_t pos, int32_t* start, int32_t* end) {
    int64_t a, b;
    visible_keys(ctx, layer, pos, &a, &b);
    *start = (int32_t)a;
    *end = (int32_t)b;
}

// call site src/engine/runtime/inference.rs:3499-3507, once per sequence
void ora_decode(ora_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q, const float* k,
                const float* v, float* out) {
    std::vector<float> qb(ctx->q_dim), kb(ctx->kv_dim), vb(ctx->kv_dim);
    for (int b = 0; b < B; ++b) {
        std::memcpy(qb.data(), q + (size_t)b * ctx->q_dim, sizeof(float) * ctx->q_dim);
        std::memcpy(kb.data(), k + (size_t)b * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        std::memcpy(vb.data(), v + (size_t)b * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        qkv_bias_and_norm(ctx, layer, qb.data(), kb.data(), vb.data());
        apply_rope(ctx, layer, pos[b], qb.data(), kb.data());
        kv_write(ctx, b, layer, pos[b], kb.data(), vb.data());
        attention_token(ctx, b, layer, pos[b], qb.data(), out + (size_t)b * ctx->q_dim);
    }
}

// call site src/engine/runtime/inference.rs:2981-3017 (attention part)
void ora_prefill(ora_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const float* q,
                 const float* k, const float* v, float* out) {
    std::vector<float> qb(ctx->q_dim), kb(ctx->kv_dim), vb(ctx->kv_dim);
    for (int i = 0; i < m; ++i) {
        int pos = base_pos + i;
        std::memcpy(qb.data(), q + (size_t)i * ctx->q_dim, sizeof(float) * ctx->q_dim);
        std::memcpy(kb.data(), k + (size_t)i * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        std::memcpy(vb.data(), v + (size_t)i * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        qkv_bias_and_norm(ctx, layer, qb.data(), kb.data(), vb.data());
        apply_rope(ctx, layer, pos, qb.data(), kb.data());
        kv_write(ctx, seq, layer, pos, kb.data(), vb.data());
        attention_token(ctx, seq, layer, pos, qb.data(), out + (size_t)i * ctx->q_dim);
    }
}

// call site src/engine/runtime/media_prefill.rs:87-118 (attention part)
void ora_prefill_block(ora_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const float* q,
                       const float* k, const float* v, float* out) {
    std::vector<float> queries((size_t)m * ctx->q_dim), kb(ctx->kv_dim), vb(ctx->kv_dim);
    std::memcpy(queries.data(), q, sizeof(float) * (size_t)m * ctx->q_dim);
    for (int i = 0; i < m; ++i) {
        int pos = base_pos + i;
        std::memcpy(kb.data(), k + (size_t)i * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        std::memcpy(vb.data(), v + (size_t)i * ctx->kv_dim, sizeof(float) * ctx->kv_dim);
        qkv_bias_and_norm(ctx, layer, queries.data() + (size_t)i * ctx->q_dim, kb.data(), vb.data());
        apply_rope(ctx, layer, pos, queries.data() + (size_t)i * ctx->q_dim, kb.data());
        kv_write(ctx, seq, layer, pos, kb.data(), vb.data());
    }
    for (int i = 0; i < m; ++i)
        attention_token(ctx, seq, layer, base_pos + i, queries.data() + (size_t)i * ctx->q_dim,
                        out + (size_t)i * ctx->q_dim);
}

void ora_kv_read_row(ora_ctx* s, int32_t seq, int32_t layer, int32_t pos, float* k_out, float* v_out) {
    size_t r = row_index(s, seq, layer, pos), off = r * s->kv_dim;
    for (int i = 0; i < s->kv_dim; ++i) {
        switch (s->c.kv_format) {
            case 0:
                k_out[i] = s->kf[off + i];
                v_out[i] = s->vf[off + i];
                break;
            case 1:
                k_out[i] = bf16_to_f32(s->kh[off + i]);
                v_out[i] = bf16_to_f32(s->vh[off + i]);
                break;
            case 2:
                k_out[i] = (float)s->kq[off + i] * s->ks[r];
                v_out[i] = (float)s->vq[off + i] * s->vs[r];
                break;
            case 3: {
                int nb = s->kv_dim / 32;
                k_out[i] = (float)s->kq[off + i] * s->ks[r * nb + i / 32];
                v_out[i] = (float)s->vq[off + i] * s->vs[r * nb + i / 32];
                break;
            }
        }
    }
}

// raw TurboQuant row: codes (kv_dim / 4 bytes), sign bits (kv_dim / 8 bytes), sigma and residual norm per kv head
int ora_kv_read_turbo(ora_ctx* s, int32_t seq, int32_t layer, int32_t pos, uint8_t* k_base, uint8_t* v_base,
                      uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale, float* k_rnorm, float* v_rnorm) {
    if (s->c.kv_format != 4 || s->kv_dim % 8 != 0) return -1;
    size_t r = row_index(s, seq, layer, pos), off = r * s->kv_dim;
    std::memcpy(k_base, &s->kt_base[off / 4], s->kv_dim / 4);
    std::memcpy(v_base, &s->vt_base[off / 4], s->kv_dim / 4);
    std::memcpy(k_sign, &s->kt_sign[off / 8], s->kv_dim / 8);
    std::memcpy(v_sign, &s->vt_sign[off / 8], s->kv_dim / 8);
    for (int h = 0; h < s->c.n_kv_heads; ++h) {
        size_t aux = r * s->c.n_kv_heads + h;
        k_scale[h] = s->ks[aux];
        v_scale[h] = s->vs[aux];
        k_rnorm[h] = s->k_rnorm[aux];
        v_rnorm[h] = s->v_rnorm[aux];
    }
    return 0;
}

// the transform of the reference's property tests (:4546-4566): signs of slot `first`, FWHT, signs of slot `second`
int ora_turbo_transform(ora_ctx* s, int32_t layer, int32_t kv_head, int32_t first_slot, int32_t second_slot, float* values) {
    if (s->c.kv_format != 4 || first_slot < 0 || first_slot > 3 || second_slot < 0 || second_slot > 3) return -1;
    turbo_transform(values, s->D, turbo_sign_slot(s, first_slot, layer, kv_head), turbo_sign_slot(s, second_slot, layer, kv_head));
    return 0;
}

int ora_kv_read_q8(ora_ctx* s, int32_t seq, int32_t layer, int32_t pos, int8_t* k_q, int8_t* v_q, float* k_scale,
                   float* v_scale) {
    if (s->c.kv_format != 2 && s->c.kv_format != 3) return -1;
    size_t r = row_index(s, seq, layer, pos), off = r * s->kv_dim;
    std::memcpy(k_q, &s->kq[off], s->kv_dim);
    std::memcpy(v_q, &s->vq[off], s->kv_dim);
    int ns = s->c.kv_format == 2 ? 1 : s->kv_dim / 32;
    for (int i = 0; i < ns; ++i) {
        k_scale[i] = s->ks[r * ns + i];
        v_scale[i] = s->vs[r * ns + i];
    }
    return 0;
}

ora_plan* ora_plan_new(void) { return new ora_plan(); }
void ora_plan_free(ora_plan* p) { delete p; }

// src/engine/positions.rs:4-13
int ora_plan_append_text(ora_plan* p, int64_t count) {
    if (count < 0 || count > std::numeric_limits<int64_t>::max() - p->next_text) return -1;
    int64_t end = p->next_text + count;
    for (int64_t v = p->next_text; v < end; ++v) p->positions.push_back({v, v, v});
    p->next_text = end;
    return 0;
}

// src/engine/positions.rs:16-44
int ora_plan_append_grid(ora_plan* p, int64_t t, int64_t h, int64_t w, int64_t token_count) {
    if (t < 0 || h < 0 || w < 0) return -1;
    __int128 count = (__int128)t * h;
    if (count > std::numeric_limits<int64_t>::max()) return -1;
    count *= w;
    if (count > std::numeric_limits<int64_t>::max()) return -1;
    if (count == 0 || (int64_t)count != token_count) return -1;
    int64_t base = p->next_text;
    int64_t mx = std::max(t, std::max(h, w));
    if (mx > std::numeric_limits<int64_t>::max() - base) return -1;
    for (int64_t a = 0; a < t; ++a)
        for (int64_t b = 0; b < h; ++b)
            for (int64_t c = 0; c < w; ++c) p->positions.push_back({base + a, base + b, base + c});
    p->next_text = base + mx;
    return 0;
}

int64_t ora_plan_len(const ora_plan* p) { return (int64_t)p->positions.size(); }
int64_t ora_plan_next_text(const ora_plan* p) { return p->next_text; }
void ora_plan_at(const ora_plan* p, int64_t pos, int64_t out[3]) { plan_at(*p, pos, out); }
int32_t ora_rope_axis(int32_t layout, int32_t frequency, const int32_t sections[4]) {
    return rope_axis(layout, frequency, sections);
}

// src/vendors/gemma.rs:92-100 (scalar period form; 0 = every layer local)
int ora_gemma_layer_windows(int32_t n_layers, int32_t window, int32_t period, int32_t* out) {
    for (int l = 0; l < n_layers; ++l) {
        bool local = window > 0 && (period == 0 || l % period != period - 1);
        out[l] = local ? window : 0;
    }
    return 0;
}

uint16_t ora_f32_to_bf16(float x) { return f32_to_bf16(x); }
float ora_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

}  // extern "C"
