//! Raw FFI declarations and a small owning wrapper for `libggr_attn.so`, the B200 (sm_100a) attention path
//! of gguf-runner. The declarations mirror `include/ggr_attn.h` one to one (same order); the wrapper is what
//! `RunState` would hold in place of its KV-cache vectors.
//!
//! Status codes never abort: every call returns `ggr_status`, and `GpuAttn::check` turns a nonzero status into
//! the `Err(String)` the engine's attention half-layer already propagates.
#![allow(clippy::too_many_arguments)]

use core::ffi::{c_char, c_void};
use std::ffi::CStr;

pub const GGR_ATTN_ABI_VERSION: i32 = 2;

pub const GGR_OK: i32 = 0;
pub const GGR_ERR_INVALID: i32 = 1;
pub const GGR_ERR_CUDA: i32 = 2;
pub const GGR_ERR_ALLOC: i32 = 3;
pub const GGR_ERR_RANGE: i32 = 4;
pub const GGR_ERR_UNSUPPORTED: i32 = 5;
pub const GGR_ERR_TIMEOUT: i32 = 6;
pub const GGR_ERR_COMM: i32 = 7;

pub const GGR_PTR_HOST: i32 = 0;
pub const GGR_PTR_DEVICE: i32 = 1;
pub const GGR_DTYPE_F32: i32 = 0;
pub const GGR_DTYPE_BF16: i32 = 1;
pub const GGR_KV_F32: i32 = 0;
pub const GGR_KV_BF16: i32 = 1;
pub const GGR_KV_Q8_ROW: i32 = 2;
pub const GGR_KV_Q8_BLOCK32: i32 = 3;
pub const GGR_KV_TURBO: i32 = 4;
pub const GGR_ROPE_NEOX: i32 = 0;
pub const GGR_ROPE_ADJACENT: i32 = 1;
pub const GGR_ROPE_SEQUENTIAL: i32 = 0;
pub const GGR_ROPE_INTERLEAVED: i32 = 1;
pub const GGR_SCALE_SCORE: i32 = 0;
pub const GGR_SCALE_Q_PRESCALED: i32 = 1;
pub const GGR_IMAGE_CAUSAL: i32 = 0;
pub const GGR_IMAGE_BIDIRECTIONAL: i32 = 1;
pub const GGR_SHARD_NONE: i32 = 0;
pub const GGR_SHARD_KV_SEQUENCE: i32 = 2;
pub const GGR_IMPL_AUTO: i32 = 0;
pub const GGR_IMPL_SIMT: i32 = 1;
pub const GGR_IMPL_MMA: i32 = 2;
pub const GGR_IMPL_TCGEN05: i32 = 3;

/// `ggr_attn_config`: field order and types follow the C struct exactly.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct GgrAttnConfig {
    pub struct_size: i32,
    pub n_layers: i32,
    pub n_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub rope_dim: i32,
    pub seq_len: i32,
    pub max_batch: i32,
    pub rope_theta: f32,
    pub rope_theta_swa: f32,
    pub rope_scale_global: f32,
    pub rope_scale_local: f32,
    pub rope_style: i32,
    pub rope_layout: i32,
    pub rope_sections: [i32; 4],
    pub swa_theta_on_window_layers: i32,
    pub swa_pattern: i32,
    pub scale_mode: i32,
    pub softmax_mode: i32,
    pub kv_format: i32,
    pub image_mode: i32,
    pub n_layer_windows: i32,
    pub layer_windows: *const i32,
    pub device: i32,
    pub shard_mode: i32,
    pub shard_pos_begin: i32,
    pub shard_pos_count: i32,
    pub n_ranks: i32,
    pub rank: i32,
    pub decode_impl: i32,
    pub prefill_impl: i32,
    pub max_splits: i32,
    pub decode_fusion: i32,
    pub exchange_wait_us: i32,
}

#[repr(C)]
pub struct GgrAttnCtx {
    _private: [u8; 0],
}

#[repr(C)]
pub struct GgrRopePlan {
    _private: [u8; 0],
}

#[repr(C)]
pub struct GgrWeights {
    _private: [u8; 0],
}

pub const GGR_W_F32: i32 = 0;
pub const GGR_W_BF16: i32 = 1;
pub const GGR_W_Q8_0: i32 = 2;
pub const GGR_W_Q4_K: i32 = 3;
pub const GGR_W_Q6_K: i32 = 4;

#[link(name = "ggr_attn")]
extern "C" {
    pub fn ggr_attn_config_init(cfg: *mut GgrAttnConfig);
    pub fn ggr_attn_create(cfg: *const GgrAttnConfig, out: *mut *mut GgrAttnCtx) -> i32;
    pub fn ggr_attn_destroy(ctx: *mut GgrAttnCtx);
    pub fn ggr_attn_last_error(ctx: *const GgrAttnCtx) -> *const c_char;
    pub fn ggr_attn_create_error() -> *const c_char;
    pub fn ggr_attn_abi_version() -> i32;
    pub fn ggr_attn_set_stream(ctx: *mut GgrAttnCtx, cuda_stream: *mut c_void) -> i32;
    pub fn ggr_attn_synchronize(ctx: *mut GgrAttnCtx) -> i32;
    pub fn ggr_attn_set_position_plan(ctx: *mut GgrAttnCtx, thw: *const i32, n: i32, next_text_pos: i32) -> i32;
    pub fn ggr_attn_set_media_blocks(ctx: *mut GgrAttnCtx, start_len: *const i32, n: i32, prompt_tokens: i32) -> i32;
    pub fn ggr_attn_visible_keys(ctx: *const GgrAttnCtx, layer: i32, pos: i32, start: *mut i32,
        end: *mut i32) -> i32;
    pub fn ggr_attn_set_layer_fixups(ctx: *mut GgrAttnCtx, layer: i32, q_bias: *const f32,
        k_bias: *const f32, v_bias: *const f32, q_norm: *const f32, k_norm: *const f32, eps: f32) -> i32;
    pub fn ggr_attn_decode(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, q: *const f32,
        k: *const f32, v: *const f32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_decode_gated(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, q: *const f32,
        k: *const f32, v: *const f32, gate: *const f32, gate_head_stride: i32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_reserve(ctx: *mut GgrAttnCtx, b: i32) -> i32;
    pub fn ggr_attn_prefill(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, base_pos: i32, m: i32,
        q: *const c_void, k: *const c_void, v: *const c_void, in_dtype: i32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_prefill_gated(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, base_pos: i32, m: i32,
        q: *const c_void, k: *const c_void, v: *const c_void, gate: *const c_void, gate_head_stride: i32,
        in_dtype: i32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_prefill_block(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, base_pos: i32, m: i32,
        q: *const c_void, k: *const c_void, v: *const c_void, in_dtype: i32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_apply_rope_qk(ctx: *mut GgrAttnCtx, layer: i32, pos: i32, q: *mut f32, k: *mut f32,
        ptr_kind: i32) -> i32;
    pub fn ggr_attn_kv_write_token(ctx: *mut GgrAttnCtx, seq: i32, layer: i32, pos: i32, k: *const f32,
        v: *const f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_attention_token(ctx: *mut GgrAttnCtx, seq: i32, layer: i32, pos: i32, q: *const f32,
        out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_decode_partial(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, q: *const f32,
        k: *const f32, v: *const f32, partial: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_combine_partials(ctx: *mut GgrAttnCtx, parts: *const f32, n_parts: i32, b: i32,
        out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_exchange_create(ctx: *mut GgrAttnCtx, max_b: i32, local_base: *mut *mut c_void,
        ipc_handle: *mut u8) -> i32;
    pub fn ggr_attn_exchange_connect(ctx: *mut GgrAttnCtx, ipc_handles: *const u8,
        same_process_ptrs: *const *mut c_void) -> i32;
    pub fn ggr_attn_decode_exchange(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, q: *const f32,
        k: *const f32, v: *const f32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_exchange_send(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, q: *const f32,
        k: *const f32, v: *const f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_exchange_receive(ctx: *mut GgrAttnCtx, b: i32, out: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_exchange_epoch(ctx: *const GgrAttnCtx) -> i32;
    pub fn ggr_attn_exchange_resync(ctx: *mut GgrAttnCtx, epoch: i32) -> i32;
    pub fn ggr_attn_kv_export(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, row0: i32, nrows: i32,
        k_q8: *mut i8, v_q8: *mut i8, k_scale: *mut f32, v_scale: *mut f32) -> i32;
    pub fn ggr_attn_kv_import(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, row0: i32, nrows: i32,
        k_q8: *const i8, v_q8: *const i8, k_scale: *const f32, v_scale: *const f32) -> i32;
    pub fn ggr_attn_kv_export_turbo(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, row0: i32, nrows: i32,
        k_base: *mut u8, v_base: *mut u8, k_sign: *mut u8, v_sign: *mut u8, k_scale: *mut f32,
        v_scale: *mut f32, k_rnorm: *mut f32, v_rnorm: *mut f32) -> i32;
    pub fn ggr_attn_kv_import_turbo(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, row0: i32, nrows: i32,
        k_base: *const u8, v_base: *const u8, k_sign: *const u8, v_sign: *const u8, k_scale: *const f32,
        v_scale: *const f32, k_rnorm: *const f32, v_rnorm: *const f32) -> i32;
    pub fn ggr_attn_kv_read_row(ctx: *mut GgrAttnCtx, seq: i32, layer: i32, pos: i32, k_out: *mut f32,
        v_out: *mut f32) -> i32;
    pub fn ggr_attn_kv_read_turbo(ctx: *mut GgrAttnCtx, seq: i32, layer: i32, pos: i32, k_base: *mut u8,
        v_base: *mut u8, k_sign: *mut u8, v_sign: *mut u8, k_scale: *mut f32, v_scale: *mut f32,
        k_rnorm: *mut f32, v_rnorm: *mut f32) -> i32;
    pub fn ggr_attn_attention_tokens_static(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32,
        q_dev: *const f32, out_dev: *mut f32) -> i32;
    pub fn ggr_weights_upload(device: i32, wtype: i32, rows: i32, cols: i32, host_data: *const c_void,
        out: *mut *mut GgrWeights) -> i32;
    pub fn ggr_weights_free(w: *mut GgrWeights);
    pub fn ggr_proj_matmul(ctx: *mut GgrAttnCtx, w: *const GgrWeights, x: *const f32, n: i32, xout: *mut f32,
        ptr_kind: i32) -> i32;
    pub fn ggr_attn_layer_decode(ctx: *mut GgrAttnCtx, layer: i32, pos: *const i32, b: i32, xb: *const f32,
        wq: *const GgrWeights, wk: *const GgrWeights, wv: *const GgrWeights, wo: *const GgrWeights,
        xb2: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_layer_prefill(ctx: *mut GgrAttnCtx, layer: i32, seq: i32, base_pos: i32, m: i32,
        xb: *const f32, wq: *const GgrWeights, wk: *const GgrWeights, wv: *const GgrWeights,
        wo: *const GgrWeights, xb2: *mut f32, ptr_kind: i32) -> i32;
    pub fn ggr_attn_launch_count(ctx: *const GgrAttnCtx) -> i64;
    pub fn ggr_attn_last_split_count(ctx: *const GgrAttnCtx) -> i32;
    pub fn ggr_attn_set_kernel_timing(ctx: *mut GgrAttnCtx, enable: i32) -> i32;
    pub fn ggr_attn_kernel_time(ctx: *mut GgrAttnCtx, kind: i32, total_ms: *mut f64, launches: *mut i64,
        reset: i32) -> i32;
    pub fn ggr_attn_kv_device_ptrs(ctx: *mut GgrAttnCtx, k: *mut *mut c_void, v: *mut *mut c_void,
        k_scale: *mut *mut f32, v_scale: *mut *mut f32, array_bytes: *mut u64) -> i32;
    pub fn ggr_rope_plan_new() -> *mut GgrRopePlan;
    pub fn ggr_rope_plan_free(plan: *mut GgrRopePlan);
    pub fn ggr_rope_plan_append_text(plan: *mut GgrRopePlan, count: i64) -> i32;
    pub fn ggr_rope_plan_append_grid(plan: *mut GgrRopePlan, t: i64, h: i64, w: i64, token_count: i64) -> i32;
    pub fn ggr_rope_plan_len(plan: *const GgrRopePlan) -> i64;
    pub fn ggr_rope_plan_next_text(plan: *const GgrRopePlan) -> i64;
    pub fn ggr_rope_plan_at(plan: *const GgrRopePlan, pos: i64, out: *mut i64);
    pub fn ggr_rope_plan_export(plan: *const GgrRopePlan, out: *mut i32, n: i64) -> i64;
    pub fn ggr_rope_axis(layout: i32, frequency: i32, sections: *const i32) -> i32;
    pub fn ggr_media_plan_validate(start_len: *const i64, n: i32, prompt_tokens: i64) -> i32;
    pub fn ggr_media_chunk_end(start_len: *const i64, n: i32, prompt_tokens: i64, start: i64, limit: i64,
        chunk: i64) -> i64;
    pub fn ggr_gemma_layer_windows(n_layers: i32, window: i32, period: i32, out: *mut i32) -> i32;
}

/// Owner of one device KV cache: the KV half of `RunState`, created where
/// `malloc_run_state_with_kv_cache_format` sizes the cache and dropped with the `RunState`.
pub struct GpuAttn {
    pub ctx: *mut GgrAttnCtx,
}

// One context is driven by the thread that owns its RunState; contexts are independent of each other.
unsafe impl Send for GpuAttn {}

impl GpuAttn {
    /// `windows` is empty or holds one entry per layer (0 = global), as in `LanguageAttentionPolicy::layer_windows`.
    pub fn new(mut cfg: GgrAttnConfig, windows: &[i32]) -> Result<Self, String> {
        cfg.struct_size = core::mem::size_of::<GgrAttnConfig>() as i32;
        cfg.n_layer_windows = windows.len() as i32;
        cfg.layer_windows = if windows.is_empty() { core::ptr::null() } else { windows.as_ptr() };
        let mut ctx: *mut GgrAttnCtx = core::ptr::null_mut();
        let status = unsafe { ggr_attn_create(&cfg, &mut ctx) };
        if status != GGR_OK {
            let msg = unsafe { CStr::from_ptr(ggr_attn_create_error()) }.to_string_lossy().into_owned();
            return Err(format!("ggr_attn_create failed ({status}): {msg}"));
        }
        Ok(Self { ctx })
    }

    /// A config filled with the reference's defaults (`ggr_attn_config_init`).
    pub fn default_config() -> GgrAttnConfig {
        let mut cfg = core::mem::MaybeUninit::<GgrAttnConfig>::zeroed();
        unsafe {
            ggr_attn_config_init(cfg.as_mut_ptr());
            cfg.assume_init()
        }
    }

    /// Maps a status to the `Result<(), String>` the engine's callers propagate.
    pub fn check(&self, status: i32) -> Result<(), String> {
        if status == GGR_OK {
            return Ok(());
        }
        let msg = unsafe { CStr::from_ptr(ggr_attn_last_error(self.ctx)) }.to_string_lossy().into_owned();
        Err(format!("attention path failed ({status}): {msg}"))
    }

    /// rope -> append -> attend for one token (call site `layer_attention_token_staged`).
    pub fn decode_token(&self, layer: usize, pos: usize, q: &[f32], k: &[f32], v: &[f32], out: &mut [f32]) -> Result<(), String> {
        let pos32 = [pos as i32];
        self.check(unsafe {
            ggr_attn_decode(self.ctx, layer as i32, pos32.as_ptr(), 1, q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_mut_ptr(),
                            GGR_PTR_HOST)
        })
    }

    /// The per-token loop of `transformer_prefill_batch` for `m` rows starting at `base_pos`.
    pub fn prefill_rows(&self, layer: usize, base_pos: usize, m: usize, q: &[f32], k: &[f32], v: &[f32],
                        out: &mut [f32]) -> Result<(), String> {
        self.check(unsafe {
            ggr_attn_prefill(self.ctx, layer as i32, 0, base_pos as i32, m as i32, q.as_ptr().cast(), k.as_ptr().cast(),
                             v.as_ptr().cast(), GGR_DTYPE_F32, out.as_mut_ptr(), GGR_PTR_HOST)
        })
    }

    /// Both passes of `transformer_prefill_image_block` for one complete block.
    pub fn prefill_image_block(&self, layer: usize, base_pos: usize, m: usize, q: &[f32], k: &[f32], v: &[f32],
                               out: &mut [f32]) -> Result<(), String> {
        self.check(unsafe {
            ggr_attn_prefill_block(self.ctx, layer as i32, 0, base_pos as i32, m as i32, q.as_ptr().cast(),
                                   k.as_ptr().cast(), v.as_ptr().cast(), GGR_DTYPE_F32, out.as_mut_ptr(), GGR_PTR_HOST)
        })
    }
}

impl Drop for GpuAttn {
    fn drop(&mut self) {
        if !self.ctx.is_null() {
            unsafe { ggr_attn_destroy(self.ctx) };
            self.ctx = core::ptr::null_mut();
        }
    }
}
