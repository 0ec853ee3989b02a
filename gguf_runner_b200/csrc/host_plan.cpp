// Host-side planners of the attention path: logical RoPE positions, image
// block validation and chunk boundaries, window lists. Integer logic only; it
// needs no device. Each function names the reference lines it stands for
// (paths inside apimeister/gguf-runner).
#include <algorithm>
#include <array>
#include <cstdint>
#include <limits>
#include <vector>

#include "../../include/ggr_attn.h"

struct ggr_rope_plan {
    std::vector<std::array<int64_t, 3>> positions;
    int64_t next_text_position = 0;
};

namespace {
constexpr int64_t kMax = std::numeric_limits<int64_t>::max();

// index of the block holding `position`, or -1 (MediaAttentionPlan::block_at,
// src/engine/runtime/attention.rs:30-39)
int block_index(const int64_t* sl, int32_t n, int64_t position) {
    // partition point of token_start <= position
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) / 2;
        if (sl[2 * mid] <= position)
            lo = mid + 1;
        else
            hi = mid;
    }
    if (lo == 0) return -1;
    int i = lo - 1;
    return (position - sl[2 * i] < sl[2 * i + 1]) ? i : -1;
}
}  // namespace

extern "C" {

ggr_rope_plan* ggr_rope_plan_new(void) { return new ggr_rope_plan(); }
void ggr_rope_plan_free(ggr_rope_plan* plan) { delete plan; }

int ggr_rope_plan_append_text(ggr_rope_plan* plan, int64_t count) {
    if (!plan || count < 0 || count > kMax - plan->next_text_position) return GGR_ERR_INVALID;
    const int64_t end = plan->next_text_position + count;
    plan->positions.reserve(plan->positions.size() + (size_t)count);
    for (int64_t p = plan->next_text_position; p < end; ++p) plan->positions.push_back({p, p, p});
    plan->next_text_position = end;
    return GGR_OK;
}

int ggr_rope_plan_append_grid(ggr_rope_plan* plan, int64_t t, int64_t h, int64_t w, int64_t token_count) {
    if (!plan || t < 0 || h < 0 || w < 0) return GGR_ERR_INVALID;
    // checked product, as the reference's checked_mul chain
    if (t != 0 && h > kMax / t) return GGR_ERR_INVALID;
    const int64_t th = t * h;
    if (th != 0 && w > kMax / th) return GGR_ERR_INVALID;
    const int64_t count = th * w;
    if (count == 0 || count != token_count) return GGR_ERR_INVALID;
    const int64_t base = plan->next_text_position;
    const int64_t span = std::max(t, std::max(h, w));
    if (span > kMax - base) return GGR_ERR_INVALID;
    plan->positions.reserve(plan->positions.size() + (size_t)count);
    for (int64_t a = 0; a < t; ++a)
        for (int64_t b = 0; b < h; ++b)
            for (int64_t c = 0; c < w; ++c) plan->positions.push_back({base + a, base + b, base + c});
    plan->next_text_position = base + span;
    return GGR_OK;
}

int64_t ggr_rope_plan_len(const ggr_rope_plan* plan) { return (int64_t)plan->positions.size(); }
int64_t ggr_rope_plan_next_text(const ggr_rope_plan* plan) { return plan->next_text_position; }

void ggr_rope_plan_at(const ggr_rope_plan* plan, int64_t pos, int64_t out[3]) {
    if (pos >= 0 && (uint64_t)pos < plan->positions.size()) {
        for (int i = 0; i < 3; ++i) out[i] = plan->positions[(size_t)pos][i];
        return;
    }
    const int64_t v = plan->next_text_position + (pos - (int64_t)plan->positions.size());
    out[0] = out[1] = out[2] = v;
}

int64_t ggr_rope_plan_export(const ggr_rope_plan* plan, int32_t* out, int64_t n) {
    const int64_t rows = std::min<int64_t>(n, (int64_t)plan->positions.size());
    for (int64_t r = 0; r < rows; ++r)
        for (int i = 0; i < 3; ++i) out[3 * r + i] = (int32_t)plan->positions[(size_t)r][i];
    return rows;
}

int32_t ggr_rope_axis(int32_t layout, int32_t frequency, const int32_t sections[4]) {
    if (layout != GGR_ROPE_INTERLEAVED) return 0;
    const int32_t axis = frequency % 3;
    return (axis != 0 && frequency / 3 < sections[axis]) ? axis : 0;
}

int ggr_media_plan_validate(const int64_t* start_len, int32_t n, int64_t prompt_tokens) {
    int64_t previous_end = 0;
    for (int32_t i = 0; i < n; ++i) {
        const int64_t start = start_len[2 * i], len = start_len[2 * i + 1];
        if (start < 0 || len < 0 || len > kMax - start) return GGR_ERR_INVALID;  // range overflow
        const int64_t end = start + len;
        if (len == 0 || start < previous_end || end > prompt_tokens) return GGR_ERR_INVALID;
        previous_end = end;
    }
    return GGR_OK;
}

int64_t ggr_media_chunk_end(const int64_t* start_len, int32_t n, int64_t prompt_tokens, int64_t start,
                            int64_t limit, int64_t chunk) {
    if (chunk <= 0 || start >= limit || limit > prompt_tokens) return -(int64_t)GGR_ERR_INVALID;
    const int bi = block_index(start_len, n, start);
    if (bi >= 0) {
        const int64_t bs = start_len[2 * bi], end = bs + start_len[2 * bi + 1];
        if (start != bs) return -(int64_t)GGR_ERR_INVALID;  // cannot resume inside an image block
        if (end > limit) return -(int64_t)GGR_ERR_INVALID;  // limit splits an image block
        return end;
    }
    int64_t end = chunk > kMax - start ? kMax : start + chunk;  // saturating add
    end = std::min(end, limit);
    for (int32_t i = 0; i < n; ++i)
        if (start_len[2 * i] >= start && start_len[2 * i] < end) return start_len[2 * i];
    return end;
}

int ggr_gemma_layer_windows(int32_t n_layers, int32_t window, int32_t period, int32_t* out) {
    if (n_layers < 0 || window < 0 || period < 0 || !out) return GGR_ERR_INVALID;
    for (int32_t l = 0; l < n_layers; ++l) {
        const bool local = window > 0 && (period == 0 || l % period != period - 1);
        out[l] = local ? window : 0;
    }
    return GGR_OK;
}

}  // extern "C"

// ---- TurboQuant transform signs (src/engine/runtime/inference.rs:370-395, splitmix64 :673-679) ----

namespace {
inline uint64_t turbo_splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
}  // namespace

// Sign bits of the four transforms {rot_pre, rot_post, res_pre, res_post} for every (layer, kv head):
// layout [slot][layer][kv_head][ceil(D / 8)], element i is negated iff its bit (LSB first) is set.
std::vector<unsigned char> ggr_turbo_sign_table(int n_layers, int n_kv_heads, int head_dim) {
    static const uint64_t salts[4] = {0x9E3779B97F4A7C15ull, 0xC2B2AE3D27D4EB4Full, 0x165667B19E3779F9ull,
                                      0xD6E8FEB86659FD93ull};
    const size_t bytes = (size_t)(head_dim + 7) / 8, stride = (size_t)n_layers * n_kv_heads * bytes;
    std::vector<unsigned char> table(4 * stride, 0);
    for (int slot = 0; slot < 4; ++slot)
        for (int l = 0; l < n_layers; ++l)
            for (int h = 0; h < n_kv_heads; ++h) {
                const uint64_t seed = turbo_splitmix64(((uint64_t)l << 32) ^ (uint64_t)h ^ salts[slot]);
                unsigned char* bits = &table[slot * stride + ((size_t)l * n_kv_heads + h) * bytes];
                for (int i = 0; i < head_dim; ++i)
                    if (turbo_splitmix64(seed ^ (uint64_t)i) & 1) bits[i / 8] |= (unsigned char)(1u << (i & 7));
            }
    return table;
}

