/*
 * ggr_attn.h - C ABI of the B200 (sm_100a) attention path for gguf-runner.
 *
 * One opaque context per generation replaces the KV-cache half of the
 * reference's RunState; the entry points replace the rope -> append -> attend
 * sequence the reference runs per layer. All reference citations are paths
 * inside apimeister/gguf-runner.
 *
 * Conventions
 *  - every call returns a ggr_status; nothing aborts or traps. A nonzero
 *    status leaves a message in ggr_attn_last_error(ctx).
 *  - all pointers are caller-owned. `ptr_kind` says whether the q/k/v/out
 *    buffers of a call live in host memory (the unmodified engine: the call
 *    copies in, runs, copies out and synchronises) or in device memory (the
 *    call only enqueues work on the context's stream).
 *  - position arrays and plan tables are always host memory.
 *  - calls on one context are serialised by the caller; different contexts are
 *    independent (the reference forks one RunState per concurrent generation).
 *  - no CPU fallback exists: a missing device or a failed launch is an error.
 */
#ifndef GGR_ATTN_H
#define GGR_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GGR_ATTN_ABI_VERSION 2

typedef enum ggr_status {
    GGR_OK = 0,
    GGR_ERR_INVALID = 1,     /* bad argument or configuration */
    GGR_ERR_CUDA = 2,        /* a CUDA runtime call failed */
    GGR_ERR_ALLOC = 3,       /* device or host allocation failed */
    GGR_ERR_RANGE = 4,       /* layer / position / batch outside the cache */
    GGR_ERR_UNSUPPORTED = 5, /* shape or mode this build has no kernel for */
    GGR_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out */
    GGR_ERR_COMM = 7         /* collective setup or call failed */
} ggr_status;

enum { GGR_PTR_HOST = 0, GGR_PTR_DEVICE = 1 };
enum { GGR_DTYPE_F32 = 0, GGR_DTYPE_BF16 = 1 };
/* GGR_KV_TURBO is the reference's default cache (KvCacheFormat::Turbo, src/engine/runtime/inference.rs:1634):
 * 2-bit codes of the rotated head plus one sign bit of the projected residual per element, sigma and residual
 * norm per (row, kv head); head_dim 64, 128 or 256 */
enum { GGR_KV_F32 = 0, GGR_KV_BF16 = 1, GGR_KV_Q8_ROW = 2, GGR_KV_Q8_BLOCK32 = 3, GGR_KV_TURBO = 4 };
enum { GGR_ROPE_NEOX = 0, GGR_ROPE_ADJACENT = 1 };
enum { GGR_ROPE_SEQUENTIAL = 0, GGR_ROPE_INTERLEAVED = 1 };
enum { GGR_SCALE_SCORE = 0, GGR_SCALE_Q_PRESCALED = 1 };
enum { GGR_IMAGE_CAUSAL = 0, GGR_IMAGE_BIDIRECTIONAL = 1 };
enum { GGR_SHARD_NONE = 0, GGR_SHARD_KV_SEQUENCE = 2 };
/* decode: SIMT = CUDA cores, MMA = mma.sync fed by cp.async, AUTO = mma.sync fed by TMA where the shape allows;
 * prefill: SIMT = CUDA cores, TCGEN05 / AUTO = tcgen05 + TMEM where the shape allows */
enum { GGR_IMPL_AUTO = 0, GGR_IMPL_SIMT = 1, GGR_IMPL_MMA = 2, GGR_IMPL_TCGEN05 = 3 };

typedef struct ggr_attn_ctx ggr_attn_ctx;

/*
 * Mirrors the Config / RunState fields the reference's attention reads
 * (src/engine/types.rs:638-695, filled at src/vendors/mod.rs:906-1032 and
 * src/vendors/gemma.rs:20-106).
 */
typedef struct ggr_attn_config {
    int32_t struct_size; /* sizeof(ggr_attn_config), checked by create */
    int32_t n_layers, n_heads, n_kv_heads, head_dim;
    int32_t rope_dim;  /* 0 = head_dim (src/engine/runtime/inference.rs:1590-1594) */
    int32_t seq_len;   /* cache capacity in positions per layer and sequence */
    int32_t max_batch; /* independent sequences held by this context (reference: 1) */
    float rope_theta, rope_theta_swa; /* rope_theta_swa <= 0 selects 10000 */
    float rope_scale_global, rope_scale_local;
    int32_t rope_style;  /* GGR_ROPE_NEOX: pairs (i, i+rope_dim/2); GGR_ROPE_ADJACENT: pairs (2j, 2j+1) */
    int32_t rope_layout; /* GGR_ROPE_INTERLEAVED selects the T/H/W axis per frequency */
    int32_t rope_sections[4];
    int32_t swa_theta_on_window_layers; /* gemma3: window layers use rope_theta_swa */
    int32_t swa_pattern;  /* layer kind when layer_windows is empty: l % p < p-1 */
    int32_t scale_mode;   /* GGR_SCALE_* */
    int32_t softmax_mode; /* 0 two-pass, 1 online in the reference; the device always runs an online softmax */
    int32_t kv_format;    /* GGR_KV_* */
    int32_t image_mode;   /* GGR_IMAGE_* */
    int32_t n_layer_windows;      /* 0 or n_layers */
    const int32_t* layer_windows; /* window per layer counting the current token, 0 = global */
    int32_t device;               /* CUDA device ordinal */
    /* KV-sequence sharding (long-context decode): this context holds the
     * positions [shard_pos_begin, shard_pos_begin + shard_pos_count) of every
     * layer and sequence. shard_mode GGR_SHARD_NONE holds all of them. */
    int32_t shard_mode, shard_pos_begin, shard_pos_count;
    int32_t n_ranks, rank;
    int32_t decode_impl;  /* GGR_IMPL_*: kernel family for decode, AUTO picks by shape */
    int32_t prefill_impl; /* GGR_IMPL_*: kernel family for prefill (TurboQuant cache: GGR_IMPL_MMA moves prefill rows to
                             the tensor-core kernel, bf16-class error; default is the f32 kernel) */
    int32_t max_splits;   /* 0 = automatic split-KV factor */
    int32_t decode_fusion; /* 0 = decode rotates q and appends k/v inside the attention kernel (one launch per
                              layer) where the shape allows; 1 = separate rope/append launch */
    int32_t exchange_wait_us; /* bound, in microseconds, of the device-side wait for the peers' partial states in
                                 the fused shard exchange; 0 selects 1 000 000. On expiry the call reports
                                 GGR_ERR_TIMEOUT and the context stays usable. */
} ggr_attn_config;

/* Fills *cfg with the reference's defaults (theta 5e5, swa theta 1e4,
 * swa_pattern 6, scales 1, NeoX off ...; src/vendors/mod.rs:955-964,
 * src/vendors/llama.rs:13-15). */
void ggr_attn_config_init(ggr_attn_config* cfg);

/* Replaces malloc_run_state_with_kv_cache_format (KV and RoPE part,
 * src/engine/runtime/inference.rs:1529-1748): validates RoPE scales and the
 * window list exactly as :1533-1546, allocates the device KV cache
 * [sequence][layer][position][kv_dim] in the configured format and the RoPE
 * frequency tables. */
int ggr_attn_create(const ggr_attn_config* cfg, ggr_attn_ctx** out);
/* Replaces dropping the RunState at the end of generate_from_prefill
 * (src/app/generation.rs:4610). */
void ggr_attn_destroy(ggr_attn_ctx* ctx);
const char* ggr_attn_last_error(const ggr_attn_ctx* ctx);
/* Message of a failed ggr_attn_create (which returns no context). Thread-local. */
const char* ggr_attn_create_error(void);
int ggr_attn_abi_version(void);

/* Work of device-pointer calls is enqueued on this CUDA stream (a
 * cudaStream_t); NULL selects the non-blocking stream the context owns (the
 * default), cudaStreamLegacy the legacy default stream. */
int ggr_attn_set_stream(ggr_attn_ctx* ctx, void* cuda_stream);
int ggr_attn_synchronize(ggr_attn_ctx* ctx);

/* Replaces assigning RunState::rope_position_plan (src/app/generation.rs:4614;
 * semantics of RopePositionPlan::at, src/engine/positions.rs:46-54): thw holds
 * n rows of logical (t, h, w); rows beyond n continue at next_text_pos. n = 0
 * and next_text_pos = 0 clears the plan. */
int ggr_attn_set_position_plan(ggr_attn_ctx* ctx, const int32_t* thw, int32_t n, int32_t next_text_pos);
/* Replaces assigning RunState::media_attention_plan (src/app/generation.rs:4615-4618)
 * with the validation of MediaAttentionPlan::new (src/engine/runtime/attention.rs:9-28):
 * start_len holds n rows of (token_start, token_len). */
int ggr_attn_set_media_blocks(ggr_attn_ctx* ctx, const int32_t* start_len, int32_t n, int32_t prompt_tokens);
/* LanguageAttentionPolicy::visible_keys (src/engine/runtime/attention.rs:73-97). */
int ggr_attn_visible_keys(const ggr_attn_ctx* ctx, int32_t layer, int32_t pos, int32_t* start, int32_t* end);

/*
 * Per-layer pre-attention fixups, applied to q/k/v before RoPE inside ggr_attn_decode, ggr_attn_prefill,
 * ggr_attn_prefill_block and the shard exchange: Qwen2 q/k/v bias add and the per-head RMS norm of q and k
 * (Qwen3, Gemma3). Replaces qkv_bias_and_norm (src/engine/runtime/inference.rs:2535-2572) and
 * rmsnorm_per_head_gemma_inplace (src/engine/kernels/math.rs:164-184). Host arrays: biases [q_dim] /
 * [kv_dim] / [kv_dim] (all three or none), norm weights [head_dim] each (both or none); null clears.
 * eps <= 0 selects 1e-5 like the reference.
 */
int ggr_attn_set_layer_fixups(ggr_attn_ctx* ctx, int32_t layer, const float* q_bias, const float* k_bias,
                              const float* v_bias, const float* q_norm, const float* k_norm, float eps);

/*
 * Fused decode step: for each of B sequences, rope(q, k) + append(k, v) at
 * pos[b] + attention over the visible cache rows. Replaces the three calls at
 * src/engine/runtime/inference.rs:3499-3507 (apply_rope_qk :1817,
 * kv_write_token :1877, attention_token :1970). q is [B][n_heads*head_dim],
 * k and v are [B][n_kv_heads*head_dim] (f32, before RoPE, after bias / QK
 * norm), out is [B][n_heads*head_dim] f32, head-major like RunState::xb.
 * Sequence b of the cache belongs to batch entry b.
 */
int ggr_attn_decode(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                    const float* k, const float* v, float* out, int32_t ptr_kind);

/*
 * ggr_attn_decode followed by the Qwen3Next / Qwen3.5 output gate of the same call site
 * (src/engine/runtime/inference.rs:3509-3519: sigmoid_mul_inplace on every head, then
 * sanitize_finite_inplace): out[h][i] = finite_or_zero(attn[h][i] * sigmoid(gate[h][i])), applied in the
 * epilogue of the attention kernel. gate is f32; head h of batch entry b starts at
 * gate + (b * n_heads + h) * gate_head_stride, so the second halves of the reference's packed q / gate
 * projection (RunState::hb, head stride 2 * head_dim) can be passed as they lie; a dense [B][q_dim]
 * gate has gate_head_stride = head_dim.
 */
int ggr_attn_decode_gated(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                          const float* k, const float* v, const float* gate, int32_t gate_head_stride, float* out,
                          int32_t ptr_kind);

/*
 * Scratch reservation for decode (no counterpart in the reference, whose RunState is sized once by
 * malloc_run_state): allocates the rotated-query rows, split-KV partial states, tickets and, for host-pointer
 * calls, the pinned and device staging buffers for batches of up to B sequences, so that the decode loop that
 * follows never allocates, frees or synchronises for memory. Split-KV factors are then limited to what the
 * reservation holds. ggr_attn_create reserves for max_batch (at most 128) itself; call this only to change it.
 */
int ggr_attn_reserve(ggr_attn_ctx* ctx, int32_t B);

/*
 * Prefill of m consecutive tokens of sequence `seq` starting at base_pos;
 * token i sees exactly what attention_token would at position base_pos + i.
 * Replaces the per-token loop of transformer_prefill_batch
 * (src/engine/runtime/inference.rs:2981-3017). q/k/v are token-major
 * ([m][q_dim], [m][kv_dim]) in in_dtype; out is f32 [m][q_dim]. Like the
 * reference (:2750-2757) it rejects a chunk that overlaps a bidirectional
 * image block.
 */
int ggr_attn_prefill(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const void* q,
                     const void* k, const void* v, int32_t in_dtype, float* out, int32_t ptr_kind);

/* ggr_attn_prefill with the output gate of ggr_attn_decode_gated; gate is in in_dtype, head h of token i at
 * gate + (i * n_heads + h) * gate_head_stride. */
int ggr_attn_prefill_gated(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const void* q,
                           const void* k, const void* v, const void* gate, int32_t gate_head_stride, int32_t in_dtype,
                           float* out, int32_t ptr_kind);

/* Staged prefill of one complete image block: every row is roped and appended
 * first, then every row attends with block-wide visibility. Replaces the two
 * passes of transformer_prefill_image_block (src/engine/runtime/media_prefill.rs:87-118). */
int ggr_attn_prefill_block(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m,
                           const void* q, const void* k, const void* v, int32_t in_dtype, float* out,
                           int32_t ptr_kind);

/* The reference's three functions one by one, for callers that keep its call
 * order (and for known-answer tests). Buffers are f32. */
/* apply_rope_qk (src/engine/runtime/inference.rs:1817-1874): rotates q
 * [n_heads*head_dim] and k [n_kv_heads*head_dim] in place. */
int ggr_attn_apply_rope_qk(ggr_attn_ctx* ctx, int32_t layer, int32_t pos, float* q, float* k, int32_t ptr_kind);
/* kv_write_token (src/engine/runtime/inference.rs:1877-1918): stores an
 * already rotated k and v as cache row (seq, layer, pos). */
int ggr_attn_kv_write_token(ggr_attn_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* k,
                            const float* v, int32_t ptr_kind);
/* attention_token (src/engine/runtime/inference.rs:1970-2530): q is already
 * rotated (and pre-scaled in GGR_SCALE_Q_PRESCALED mode). */
int ggr_attn_attention_token(ggr_attn_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, const float* q,
                             float* out, int32_t ptr_kind);

/*
 * KV-sequence sharding (no counterpart in the reference, which is single
 * process): every rank holds a slab of positions, runs the fused decode over
 * its slab and emits, per (sequence, query head), a partial softmax state
 * (o[head_dim] already divided by l, m, l) with m in base-2 units
 * (score * log2 e) and l = sum 2^(s - m). The owner of pos[b] appends the
 * row. partial is [B][n_heads][head_dim + 2] f32. A rank whose slab misses
 * the visible range emits (0, -inf, 0).
 */
int ggr_attn_decode_partial(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                            const float* k, const float* v, float* partial, int32_t ptr_kind);
/* Merges n_parts partial states laid out [n_parts][B][n_heads][head_dim + 2]
 * into out [B][n_heads*head_dim]. */
int ggr_attn_combine_partials(ggr_attn_ctx* ctx, const float* parts, int32_t n_parts, int32_t B, float* out,
                              int32_t ptr_kind);

/*
 * Fused exchange for KV-sequence shards (no counterpart in the reference). Instead of all-gathering
 * the partial states with a collective, the decode kernel stores this rank's states directly into the
 * receive buffer every rank keeps (peer memory over NVLink, plain stores) and raises a flag there; a
 * second kernel waits, bounded, for all ranks' flags and merges. One call replaces
 * ggr_attn_decode_partial + all-gather + ggr_attn_combine_partials.
 *
 * ggr_attn_exchange_create allocates the local receive buffer for up to max_B sequences (uses the
 * context's n_ranks / rank, at most 8 ranks) and returns its device address and its 64-byte CUDA IPC
 * handle. ggr_attn_exchange_connect takes all ranks' handles ([n_ranks][64] bytes, gathered by the
 * host, e.g. with torch.distributed.all_gather) or, for ranks living in one process, their device
 * addresses. Every rank must make the same sequence of ggr_attn_decode_exchange calls. A rank whose
 * peers do not deliver within the bound gets GGR_ERR_TIMEOUT (after a host-pointer call, or from
 * ggr_attn_synchronize).
 */
int ggr_attn_exchange_create(ggr_attn_ctx* ctx, int32_t max_B, void** local_base, unsigned char* ipc_handle);
int ggr_attn_exchange_connect(ggr_attn_ctx* ctx, const unsigned char* ipc_handles, void* const* same_process_ptrs);
int ggr_attn_decode_exchange(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                             const float* k, const float* v, float* out, int32_t ptr_kind);
/* The two halves of ggr_attn_decode_exchange on their own: send = fused decode over the local slab with
 * the states stored to all ranks; receive = bounded wait for all ranks' states of the latest step, then
 * the merge. Ranks that share one GPU (several shards in one process) must finish every send before
 * any receive is issued, because a waiting kernel and the kernel it waits for must not depend on being
 * co-scheduled on one GPU. */
int ggr_attn_exchange_send(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* q,
                           const float* k, const float* v, int32_t ptr_kind);
int ggr_attn_exchange_receive(ggr_attn_ctx* ctx, int32_t B, float* out, int32_t ptr_kind);
/* Step counter of the exchange: the number of sends this rank has issued. A send that fails on the host
 * (before its kernel is launched) does not count. After a failed step (GGR_ERR_TIMEOUT, or a peer that
 * reported an error) the ranks agree on a value on the host (the maximum of their counters is always safe)
 * and each calls ggr_attn_exchange_resync with it; the next send then uses value + 1 on every rank. A
 * receive that finds a flag ahead of its own step reports GGR_ERR_COMM instead of merging stale states. */
int32_t ggr_attn_exchange_epoch(const ggr_attn_ctx* ctx);
int ggr_attn_exchange_resync(ggr_attn_ctx* ctx, int32_t epoch);

/* Rows [row0, row0 + nrows) of one layer of one sequence in the reference's
 * Q8 layouts, as its prefill cache serialises them (src/app/prefill_cache.rs:11-19, :214-249) and
 * re-injects them (:380-510): int8 codes [nrows][kv_dim] and, per row, one f32 scale
 * (GGR_KV_Q8_ROW, the blob's q8_block = 0) or kv_dim / 32 scales (GGR_KV_Q8_BLOCK32, q8_block = 1).
 * Host buffers. */
int ggr_attn_kv_export(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t row0, int32_t nrows, int8_t* k_q8,
                       int8_t* v_q8, float* k_scale, float* v_scale);
int ggr_attn_kv_import(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t row0, int32_t nrows,
                       const int8_t* k_q8, const int8_t* v_q8, const float* k_scale, const float* v_scale);
/* The same for the TurboQuant cache (the blob's kv_format = 1): the eight sections of
 * src/app/prefill_cache.rs:16-18 for rows [row0, row0 + nrows) of one layer: 2-bit codes
 * [nrows][kv_dim / 4], residual sign bits [nrows][kv_dim / 8], sigma and residual norm [nrows][n_kv_heads],
 * for K and for V. Host buffers; only for kv_format GGR_KV_TURBO. */
int ggr_attn_kv_export_turbo(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t row0, int32_t nrows, uint8_t* k_base,
                             uint8_t* v_base, uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale,
                             float* k_rnorm, float* v_rnorm);
int ggr_attn_kv_import_turbo(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t row0, int32_t nrows,
                             const uint8_t* k_base, const uint8_t* v_base, const uint8_t* k_sign, const uint8_t* v_sign,
                             const float* k_scale, const float* v_scale, const float* k_rnorm, const float* v_rnorm);
/* Dequantised f32 view of one cache row (any format), for tests. Host buffers. */
int ggr_attn_kv_read_row(ggr_attn_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, float* k_out, float* v_out);
/* Raw TurboQuant row in the reference's layout (src/engine/runtime/inference.rs:1919-1963): 2-bit codes
 * (kv_dim / 4 bytes, four per byte, LSB first), residual sign bits (kv_dim / 8 bytes), sigma and residual norm
 * per kv head, for K and for V. Host buffers; only for kv_format GGR_KV_TURBO. */
int ggr_attn_kv_read_turbo(ggr_attn_ctx* ctx, int32_t seq, int32_t layer, int32_t pos, uint8_t* k_base, uint8_t* v_base,
                           uint8_t* k_sign, uint8_t* v_sign, float* k_scale, float* v_scale, float* k_rnorm,
                           float* v_rnorm);

/*
 * Allocation-free variant of ggr_attn_attention_token for B sequences (no
 * counterpart in the reference, whose attention needs no scratch beyond
 * RunState::att). It is meant for hosts that cannot allocate device memory in
 * their decode loop: an engine that gave all of HBM to its caches and weights
 * at start-up, so a later cudaMalloc may fail, or one whose token loop must
 * not hit the device-wide synchronisation an allocation implies. The split-KV
 * scratch (partial softmax states and tickets) lives in a fixed 8 MiB array
 * inside the library image; every GPU that loads the library carries that
 * array until the process exits.
 *
 * q_dev is [B][n_heads*head_dim] f32, already rotated (and pre-scaled in
 * GGR_SCALE_Q_PRESCALED mode); out_dev is [B][n_heads*head_dim] f32; both are
 * device memory. Sequence b attends from position pos[b] (host array). The
 * work is enqueued on the context's stream.
 *
 * Limits: B <= 128, and two splits' worth of state, 2*B*n_heads*(head_dim+2)
 * floats, must fit in the array (about 1M floats per split); larger calls
 * return GGR_ERR_RANGE. The split count is lowered to what the array holds.
 * The first call on a device looks up the array's device address; make that
 * call before any stream capture. Calls made after that allocate nothing.
 * All contexts and calls on a device share the one array: it still holds the
 * previous call's data (the tickets are cleared at the start of each call),
 * so two such calls whose kernels overlap on the GPU race with each other;
 * issue them on one stream or order them with events.
 */
int ggr_attn_attention_tokens_static(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B,
                                     const float* q_dev, float* out_dev);

/*
 * The matmuls either side of the path, so that q / k / v never visit the host: with the projection weights
 * resident on the device a decode step moves one hidden-state row in and one out per layer instead of q, k, v
 * and the attention output.
 *
 * ggr_weights is one weight matrix [rows][cols] on a device. host_data is the tensor as the reference maps it from
 * the GGUF file (QuantizedTensor, row-major GGML rows): GGR_W_F32, GGR_W_BF16, GGR_W_Q8_0 (blocks of one f16
 * scale and 32 int8 codes, 34 bytes; src/engine/kernels/quant.rs:89, :105) or GGR_W_Q4_K (super-blocks of 256
 * weights in 144 bytes: f16 d, f16 dmin, eight packed 6-bit (scale, min) pairs, 128 bytes of nibbles;
 * dequantize_row_q4_k, src/engine/kernels/quant.rs:294-325) or GGR_W_Q6_K (super-blocks of 256 weights in 210
 * bytes: low nibbles, high bit pairs, one int8 scale per 16 weights, f16 d; dequantize_row_q6_k :484-517). cols must
 * be a multiple of 256 for the K types, of 32 for
 * Q8_0 and of 8 otherwise, rows a multiple of 8. Quantised codes and scales are kept in separate planes, and every
 * type but BF16 also keeps a bf16 image (each weight rounded once) for the tensor-core kernel that multiplies chunks
 * of rows.
 */
typedef struct ggr_weights ggr_weights;
enum { GGR_W_F32 = 0, GGR_W_BF16 = 1, GGR_W_Q8_0 = 2, GGR_W_Q4_K = 3, GGR_W_Q6_K = 4 };
int ggr_weights_upload(int32_t device, int32_t wtype, int32_t rows, int32_t cols, const void* host_data, ggr_weights** out);
void ggr_weights_free(ggr_weights* w);
/* xout[i][rows] = W x[i] for n rows of x [n][cols], f32 in and out. Replaces matmul_quantized_with_scratch
 * (src/engine/kernels/quant.rs:7225) for one row and the batched prefill matmuls of transformer_prefill_batch
 * (src/engine/runtime/inference.rs:2921-2979) for many: up to 16 rows run on a weight-streaming kernel with f32
 * arithmetic (the reference's dot of f32 activations with the decoded weights); more rows run on the tensor cores
 * with activations and weights in bf16 (tolerance of bf16 operands). */
int ggr_proj_matmul(ggr_attn_ctx* ctx, const ggr_weights* w, const float* x, int32_t n, float* xout, int32_t ptr_kind);
/*
 * The attention half of a layer for one token of each of B sequences, from the normalised hidden state to the
 * output projection: q, k, v = Wq xb, Wk xb, Wv xb (src/engine/runtime/inference.rs:3144-3476, the dense case with
 * separate projections), bias / QK-norm fixups of the layer, rope + append + attention (:3499-3507), xb2 = Wo att
 * with non-finite values zeroed (:3520-3527). xb is [B][wq.cols], xb2 is [B][wo.rows]; only these cross PCIe with
 * GGR_PTR_HOST.
 */
int ggr_attn_layer_decode(ggr_attn_ctx* ctx, int32_t layer, const int32_t* pos, int32_t B, const float* xb,
                          const ggr_weights* wq, const ggr_weights* wk, const ggr_weights* wv, const ggr_weights* wo,
                          float* xb2, int32_t ptr_kind);
/* The same for m consecutive tokens of one sequence (the attention half of transformer_prefill_batch,
 * src/engine/runtime/inference.rs:2910-3030): xb is [m][wq.cols], xb2 is [m][wo.rows]. */
int ggr_attn_layer_prefill(ggr_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t base_pos, int32_t m, const float* xb,
                           const ggr_weights* wq, const ggr_weights* wk, const ggr_weights* wv, const ggr_weights* wo,
                           float* xb2, int32_t ptr_kind);

/* Number of kernels this context has launched since it was created. */
int64_t ggr_attn_launch_count(const ggr_attn_ctx* ctx);
/* Split-KV factor the most recent decode / attention launch of this context used. */
int32_t ggr_attn_last_split_count(const ggr_attn_ctx* ctx);

/* Per-kernel device timing (the counterpart of the reference's PROF_ATTN_NS
 * counter, src/engine/profiling.rs:8-41): when enabled, every launch is
 * bracketed by CUDA events on the context's stream. kind 0 = attention
 * kernels, 1 = rope/append kernels, 2 = partial-state merges, 3 = projection matmuls.
 * ggr_attn_kernel_time synchronises the stream, returns the summed device
 * time in milliseconds and the number of launches since the last reset, and
 * resets the counters when `reset` is nonzero. */
int ggr_attn_set_kernel_timing(ggr_attn_ctx* ctx, int32_t enable);
int ggr_attn_kernel_time(ggr_attn_ctx* ctx, int32_t kind, double* total_ms, int64_t* launches, int32_t reset);

/* Device addresses of the cache arrays (layout: [sequence][layer][position -
 * shard_pos_begin][kv_dim] in the configured format; scales are null unless
 * the format is q8) and the byte size of one of the K / V arrays. For hosts
 * that keep K/V producers on the device, and for synthetic cache fills. */
int ggr_attn_kv_device_ptrs(ggr_attn_ctx* ctx, void** k, void** v, float** k_scale, float** v_scale,
                            uint64_t* array_bytes);

/* Host-side planners restated from the reference, usable without a device. */
typedef struct ggr_rope_plan ggr_rope_plan;
ggr_rope_plan* ggr_rope_plan_new(void);
void ggr_rope_plan_free(ggr_rope_plan* plan);
/* RopePositionPlan::append_text (src/engine/positions.rs:4-13) */
int ggr_rope_plan_append_text(ggr_rope_plan* plan, int64_t count);
/* RopePositionPlan::append_grid (src/engine/positions.rs:16-44) */
int ggr_rope_plan_append_grid(ggr_rope_plan* plan, int64_t t, int64_t h, int64_t w, int64_t token_count);
int64_t ggr_rope_plan_len(const ggr_rope_plan* plan);
int64_t ggr_rope_plan_next_text(const ggr_rope_plan* plan);
/* RopePositionPlan::at (src/engine/positions.rs:46-54) */
void ggr_rope_plan_at(const ggr_rope_plan* plan, int64_t pos, int64_t out[3]);
/* copies min(n, len) rows of (t, h, w) as int32 into out; returns rows copied */
int64_t ggr_rope_plan_export(const ggr_rope_plan* plan, int32_t* out, int64_t n);
/* RopePositionLayout::axis (src/engine/positions.rs:57-72) */
int32_t ggr_rope_axis(int32_t layout, int32_t frequency, const int32_t sections[4]);
/* MediaAttentionPlan::new validation (src/engine/runtime/attention.rs:9-28): 0 if valid */
int ggr_media_plan_validate(const int64_t* start_len, int32_t n, int64_t prompt_tokens);
/* MediaAttentionPlan::chunk_end (src/engine/runtime/attention.rs:43-70): end position or a negative status */
int64_t ggr_media_chunk_end(const int64_t* start_len, int32_t n, int64_t prompt_tokens, int64_t start,
                            int64_t limit, int64_t chunk);
/* Gemma3 window list from (window, period) (src/vendors/gemma.rs:92-100) */
int ggr_gemma_layer_windows(int32_t n_layers, int32_t window, int32_t period, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* GGR_ATTN_H */
