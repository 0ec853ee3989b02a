/*
 * TEST INFRASTRUCTURE - CPU oracle for the gguf-runner attention path.
 *
 * A plain C++ restatement of the reference's CPU arithmetic for RoPE, the
 * KV-cache append and causal / sliding-window GQA attention. It exists only so
 * that tests, the smoke check and the benchmark's CPU-baseline leg can compare
 * the CUDA path with it; no product code may call it.
 *
 * Pinning: the RoPE, position-plan, axis, visibility and block-validation
 * known-answer tests of the reference are restated against this oracle. The
 * numeric output of attention_token itself has no golden vector anywhere in
 * the reference, so for that function: parity unpinned (the oracle follows the
 * cited lines, but nothing from the reference's own runs checks it here; the
 * reference is Rust and no Rust toolchain exists in the build image).
 */
#ifndef GGR_ORACLE_REF_ATTENTION_H
#define GGR_ORACLE_REF_ATTENTION_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Field order mirrors the product's ggr_attn_config prefix so one ctypes
 * Structure can describe both in the tests. */
typedef struct ora_config {
    int32_t n_layers, n_heads, n_kv_heads, head_dim, rope_dim, seq_len, max_batch;
    float rope_theta, rope_theta_swa, rope_scale_global, rope_scale_local;
    int32_t rope_style;   /* 0 = NeoX split-half, 1 = adjacent pairs */
    int32_t rope_layout;  /* 0 = sequential, 1 = interleaved T/H/W */
    int32_t rope_sections[4];
    int32_t swa_theta_on_window_layers; /* gemma3: window layers use rope_theta_swa */
    int32_t swa_pattern;  /* layer-kind fallback when layer_windows is empty */
    int32_t scale_mode;   /* 0 = score *= 1/sqrt(D), 1 = q pre-scaled after RoPE */
    int32_t softmax_mode; /* 0 = two-pass, 1 = online */
    int32_t kv_format;    /* 0 f32, 1 bf16, 2 q8 row scale, 3 q8 block-32 scales, 4 TurboQuant (2 + 1 bit) */
    int32_t image_mode;   /* 0 causal, 1 bidirectional image blocks */
    int32_t n_layer_windows;
    const int32_t* layer_windows; /* n_layer_windows entries, 0 = global */
} ora_config;

typedef struct ora_ctx ora_ctx;

/* returns 0 or a negative status; *err (optional) receives a static message */
int ora_create(const ora_config* cfg, ora_ctx** out, const char** err);
void ora_destroy(ora_ctx* ctx);
void ora_set_threads(ora_ctx* ctx, int n);
int ora_threads_available(void);

int ora_set_position_plan(ora_ctx* ctx, const int32_t* thw, int32_t n, int32_t next_text_pos);
int ora_set_media_blocks(ora_ctx* ctx, const int32_t* start_len, int32_t n, int32_t prompt_tokens);

/* per-layer pre-attention fixups (null = absent): Qwen2 biases and per-head RMS QK-norm,
 * applied to q/k/v before RoPE by the call-site compositions below */
int ora_set_layer_fixups(ora_ctx* ctx, int32_t layer, const float* q_bias, const float* k_bias, const float* v_bias,
                         const float* q_norm, const float* k_norm, float eps);
void ora_qkv_bias_and_norm(ora_ctx* ctx, int32_t layer, float* q, float* k, float* v);

/* Qwen3Next / Qwen3.5 output gate on one token's attention output xb [n_heads*head_dim]: head h reads its gate at
 * gate + h * gate_head_stride (src/engine/runtime/inference.rs:3509-3519) */
void ora_sigmoid_gate(ora_ctx* ctx, float* xb, const float* gate, int32_t gate_head_stride);

/* The matmuls either side of the path, one activation row at a time (matmul_quantized_with_scratch,
 * src/engine/kernels/quant.rs:7225, scalar dots): wtype 0 = F32, 1 = BF16, 2 = Q8_0 blocks of (f16 scale, 32 int8),
 * 3 = Q4_K super-blocks of 256 (144 bytes), 4 = Q6_K super-blocks of 256 (210 bytes). */
void ora_matmul(int32_t wtype, int32_t rows, int32_t cols, const void* w, const float* x, float* xout);
float ora_fp16_to_fp32(uint16_t h);

/* the three reference functions, with explicit buffers instead of RunState */
void ora_rope_angles(ora_ctx* ctx, int32_t layer, int32_t pos, float* cos_out, float* sin_out);
void ora_apply_rope_qk(ora_ctx* ctx, int32_t layer, int32_t pos, float* q, float* k);
void ora_kv_write_token(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* k, const float* v);
void ora_attention_token(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* q, float* out);
void ora_visible_keys(ora_ctx* ctx, int32_t layer, int32_t pos, int32_t* start, int32_t* end);

/* call-site compositions: decode (one token per sequence), per-token prefill
 * loop, staged image-block prefill */
void ora_decode(ora_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q, const float* k,
                const float* v, float* out);
void ora_prefill(ora_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const float* q,
                 const float* k, const float* v, float* out);
void ora_prefill_block(ora_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const float* q,
                       const float* k, const float* v, float* out);

/* cache readers (dequantised view and raw q8 codes) for append parity */
void ora_kv_read_row(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, float* k_out, float* v_out);
int ora_kv_read_q8(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, int8_t* k_q, int8_t* v_q,
                   float* k_scale, float* v_scale);

int ora_kv_read_turbo(ora_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, uint8_t* k_base, uint8_t* v_base,
                      uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale, float* k_rnorm, float* v_rnorm);
int ora_turbo_transform(ora_ctx* ctx, int32_t layer, int32_t kv_head, int32_t first_slot, int32_t second_slot,
                        float* values);

/* host-side planners restated from the reference, for known-answer tests */
typedef struct ora_plan ora_plan;
ora_plan* ora_plan_new(void);
void ora_plan_free(ora_plan* p);
int ora_plan_append_text(ora_plan* p, int64_t count);
int ora_plan_append_grid(ora_plan* p, int64_t t, int64_t h, int64_t w, int64_t token_count);
int64_t ora_plan_len(const ora_plan* p);
int64_t ora_plan_next_text(const ora_plan* p);
void ora_plan_at(const ora_plan* p, int64_t pos, int64_t out[3]);
int32_t ora_rope_axis(int32_t layout, int32_t frequency, const int32_t sections[4]);
int ora_media_plan_validate(const int64_t* start_len, int32_t n, int64_t prompt_tokens);
int64_t ora_media_chunk_end(const int64_t* start_len, int32_t n, int64_t prompt_tokens, int64_t start,
                            int64_t limit, int64_t chunk);
int ora_gemma_layer_windows(int32_t n_layers, int32_t window, int32_t period, int32_t* out);

uint16_t ora_f32_to_bf16(float x);
float ora_bf16_to_f32(uint16_t h);

#ifdef __cplusplus
}
#endif
#endif
