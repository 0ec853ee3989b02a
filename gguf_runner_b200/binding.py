"""ctypes binding of include/ggr_attn.h.

Names follow the reference (apimeister/gguf-runner): `AttnContext.decode`
stands for the rope -> kv_write_token -> attention_token sequence at
src/engine/runtime/inference.rs:3499-3507, `prefill` for the per-token loop at
:2981-3017, `prefill_block` for src/engine/runtime/media_prefill.rs:87-118;
`apply_rope_qk`, `kv_write_token` and `attention_token` are the three reference
functions one by one. Buffers may be numpy arrays (host memory) or torch CUDA
tensors (device memory); outputs come back in the same kind.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB = None

PTR_HOST, PTR_DEVICE = 0, 1
DTYPE_F32, DTYPE_BF16 = 0, 1
KV_F32, KV_BF16, KV_Q8_ROW, KV_Q8_BLOCK32, KV_TURBO = 0, 1, 2, 3, 4
ROPE_NEOX, ROPE_ADJACENT = 0, 1
ROPE_SEQUENTIAL, ROPE_INTERLEAVED = 0, 1
SCALE_SCORE, SCALE_Q_PRESCALED = 0, 1
IMAGE_CAUSAL, IMAGE_BIDIRECTIONAL = 0, 1
SHARD_NONE, SHARD_KV_SEQUENCE = 0, 2
IMPL_AUTO, IMPL_SIMT, IMPL_MMA, IMPL_TCGEN05 = 0, 1, 2, 3

W_F32, W_BF16, W_Q8_0, W_Q4_K, W_Q6_K = 0, 1, 2, 3, 4

KV_FORMATS = {"f32": KV_F32, "bf16": KV_BF16, "q8_row": KV_Q8_ROW, "q8_block32": KV_Q8_BLOCK32, "turbo": KV_TURBO}


class GgrError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"ggr_attn status {status}: {message}")
        self.status = status
        self.message = message


class _Config(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("n_layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("rope_dim", C.c_int32), ("seq_len", C.c_int32), ("max_batch", C.c_int32),
        ("rope_theta", C.c_float), ("rope_theta_swa", C.c_float),
        ("rope_scale_global", C.c_float), ("rope_scale_local", C.c_float),
        ("rope_style", C.c_int32), ("rope_layout", C.c_int32), ("rope_sections", C.c_int32 * 4),
        ("swa_theta_on_window_layers", C.c_int32), ("swa_pattern", C.c_int32),
        ("scale_mode", C.c_int32), ("softmax_mode", C.c_int32), ("kv_format", C.c_int32),
        ("image_mode", C.c_int32), ("n_layer_windows", C.c_int32),
        ("layer_windows", C.POINTER(C.c_int32)),
        ("device", C.c_int32),
        ("shard_mode", C.c_int32), ("shard_pos_begin", C.c_int32), ("shard_pos_count", C.c_int32),
        ("n_ranks", C.c_int32), ("rank", C.c_int32),
        ("decode_impl", C.c_int32), ("prefill_impl", C.c_int32), ("max_splits", C.c_int32),
        ("decode_fusion", C.c_int32), ("exchange_wait_us", C.c_int32),
    ]


# every symbol include/ggr_attn.h declares
EXPORTED_SYMBOLS = [
    "ggr_attn_config_init", "ggr_attn_create", "ggr_attn_destroy", "ggr_attn_last_error",
    "ggr_attn_create_error", "ggr_attn_abi_version", "ggr_attn_set_stream", "ggr_attn_synchronize",
    "ggr_attn_set_position_plan", "ggr_attn_set_media_blocks", "ggr_attn_visible_keys",
    "ggr_attn_decode", "ggr_attn_prefill", "ggr_attn_prefill_block",
    "ggr_attn_apply_rope_qk", "ggr_attn_kv_write_token", "ggr_attn_attention_token",
    "ggr_attn_decode_partial", "ggr_attn_combine_partials",
    "ggr_attn_kv_export", "ggr_attn_kv_import", "ggr_attn_kv_read_row", "ggr_attn_kv_read_turbo", "ggr_attn_launch_count",
    "ggr_attn_set_kernel_timing", "ggr_attn_kernel_time", "ggr_attn_kv_device_ptrs",
    "ggr_attn_attention_tokens_static", "ggr_attn_last_split_count",
    "ggr_attn_exchange_create", "ggr_attn_exchange_connect", "ggr_attn_decode_exchange",
    "ggr_attn_exchange_send", "ggr_attn_exchange_receive", "ggr_attn_set_layer_fixups",
    "ggr_attn_exchange_epoch", "ggr_attn_exchange_resync", "ggr_attn_decode_gated", "ggr_attn_prefill_gated",
    "ggr_attn_reserve", "ggr_attn_kv_export_turbo", "ggr_attn_kv_import_turbo",
    "ggr_weights_upload", "ggr_weights_free", "ggr_proj_matmul", "ggr_attn_layer_decode", "ggr_attn_layer_prefill",
    "ggr_rope_plan_new", "ggr_rope_plan_free", "ggr_rope_plan_append_text", "ggr_rope_plan_append_grid",
    "ggr_rope_plan_len", "ggr_rope_plan_next_text", "ggr_rope_plan_at", "ggr_rope_plan_export",
    "ggr_rope_axis", "ggr_media_plan_validate", "ggr_media_chunk_end", "ggr_gemma_layer_windows",
]


def library_path() -> str:
    """libggr_attn.so beside this file; GGR_ATTN_LIBRARY names another build of the same library (e.g. the
    diagnostic build libggr_attn_trace.so, whose kernels also write phase time stamps)."""
    return os.environ.get("GGR_ATTN_LIBRARY") or os.path.join(_PKG, "libggr_attn.so")


def lib() -> C.CDLL:
    """Loads libggr_attn.so; raises if it has not been built (no fallback exists)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m gguf_runner_b200.build` "
            "(the attention path has no CPU or PyTorch fallback)")
    L = C.CDLL(path)
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    L.ggr_attn_config_init.argtypes = [C.POINTER(_Config)]
    L.ggr_attn_config_init.restype = None
    L.ggr_attn_create.argtypes = [C.POINTER(_Config), C.POINTER(vp)]
    L.ggr_attn_destroy.argtypes = [vp]
    L.ggr_attn_destroy.restype = None
    L.ggr_attn_last_error.argtypes = [vp]
    L.ggr_attn_last_error.restype = C.c_char_p
    L.ggr_attn_create_error.restype = C.c_char_p
    L.ggr_attn_set_stream.argtypes = [vp, vp]
    L.ggr_attn_synchronize.argtypes = [vp]
    L.ggr_attn_set_position_plan.argtypes = [vp, vp, i32, i32]
    L.ggr_attn_set_media_blocks.argtypes = [vp, vp, i32, i32]
    L.ggr_attn_visible_keys.argtypes = [vp, i32, i32, C.POINTER(i32), C.POINTER(i32)]
    L.ggr_attn_decode.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, i32]
    L.ggr_attn_decode_partial.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, i32]
    L.ggr_attn_combine_partials.argtypes = [vp, vp, i32, i32, vp, i32]
    L.ggr_attn_prefill.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, i32, vp, i32]
    L.ggr_attn_prefill_block.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, i32, vp, i32]
    L.ggr_attn_apply_rope_qk.argtypes = [vp, i32, i32, vp, vp, i32]
    L.ggr_attn_kv_write_token.argtypes = [vp, i32, i32, i32, vp, vp, i32]
    L.ggr_attn_attention_token.argtypes = [vp, i32, i32, i32, vp, vp, i32]
    L.ggr_attn_kv_export.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.ggr_attn_kv_import.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.ggr_attn_kv_read_row.argtypes = [vp, i32, i32, i32, vp, vp]
    L.ggr_attn_kv_read_turbo.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]
    L.ggr_attn_kv_read_turbo.restype = C.c_int
    L.ggr_attn_launch_count.argtypes = [vp]
    L.ggr_attn_launch_count.restype = i64
    L.ggr_attn_last_split_count.argtypes = [vp]
    L.ggr_attn_attention_tokens_static.argtypes = [vp, i32, vp, i32, vp, vp]
    L.ggr_attn_exchange_create.argtypes = [vp, i32, C.POINTER(vp), vp]
    L.ggr_attn_exchange_connect.argtypes = [vp, vp, vp]
    L.ggr_attn_decode_exchange.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, i32]
    L.ggr_attn_exchange_send.argtypes = [vp, i32, vp, i32, vp, vp, vp, i32]
    L.ggr_attn_exchange_receive.argtypes = [vp, i32, vp, i32]
    L.ggr_attn_set_layer_fixups.argtypes = [vp, i32, vp, vp, vp, vp, vp, C.c_float]
    L.ggr_attn_exchange_epoch.argtypes = [vp]
    L.ggr_attn_exchange_epoch.restype = i32
    L.ggr_attn_exchange_resync.argtypes = [vp, i32]
    L.ggr_attn_decode_gated.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, i32, vp, i32]
    L.ggr_attn_prefill_gated.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp, i32]
    L.ggr_attn_reserve.argtypes = [vp, i32]
    L.ggr_weights_upload.argtypes = [i32, i32, i32, i32, vp, C.POINTER(vp)]
    L.ggr_weights_free.argtypes = [vp]
    L.ggr_weights_free.restype = None
    L.ggr_proj_matmul.argtypes = [vp, vp, vp, i32, vp, i32]
    L.ggr_attn_layer_decode.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, vp, vp, i32]
    L.ggr_attn_layer_prefill.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32]
    L.ggr_attn_kv_export_turbo.argtypes = [vp, i32, i32, i32, i32] + [vp] * 8
    L.ggr_attn_kv_import_turbo.argtypes = [vp, i32, i32, i32, i32] + [vp] * 8
    L.ggr_attn_set_kernel_timing.argtypes = [vp, i32]
    L.ggr_attn_kernel_time.argtypes = [vp, i32, C.POINTER(C.c_double), C.POINTER(i64), i32]
    L.ggr_attn_kv_device_ptrs.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                          C.POINTER(C.c_uint64)]
    L.ggr_rope_plan_new.restype = vp
    L.ggr_rope_plan_free.argtypes = [vp]
    L.ggr_rope_plan_free.restype = None
    L.ggr_rope_plan_append_text.argtypes = [vp, i64]
    L.ggr_rope_plan_append_grid.argtypes = [vp, i64, i64, i64, i64]
    L.ggr_rope_plan_len.argtypes = [vp]
    L.ggr_rope_plan_len.restype = i64
    L.ggr_rope_plan_next_text.argtypes = [vp]
    L.ggr_rope_plan_next_text.restype = i64
    L.ggr_rope_plan_at.argtypes = [vp, i64, C.POINTER(i64)]
    L.ggr_rope_plan_at.restype = None
    L.ggr_rope_plan_export.argtypes = [vp, vp, i64]
    L.ggr_rope_plan_export.restype = i64
    L.ggr_rope_axis.argtypes = [i32, i32, C.POINTER(i32)]
    L.ggr_media_plan_validate.argtypes = [vp, i32, i64]
    L.ggr_media_chunk_end.argtypes = [vp, i32, i64, i64, i64, i64]
    L.ggr_media_chunk_end.restype = i64
    L.ggr_gemma_layer_windows.argtypes = [i32, i32, i32, vp]
    _LIB = L
    return L


@dataclass
class AttnConfig:
    """The Config / RunState fields the reference's attention reads (src/engine/types.rs:638-695)."""
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    seq_len: int
    max_batch: int = 1
    rope_dim: int = 0
    rope_theta: float = 500000.0
    rope_theta_swa: float = 10000.0
    rope_scale_global: float = 1.0
    rope_scale_local: float = 1.0
    rope_style: int = ROPE_NEOX
    rope_layout: int = ROPE_SEQUENTIAL
    rope_sections: Sequence[int] = (0, 0, 0, 0)
    swa_theta_on_window_layers: int = 0
    swa_pattern: int = 6
    scale_mode: int = SCALE_SCORE
    softmax_mode: int = 0
    kv_format: int = KV_Q8_ROW
    image_mode: int = IMAGE_CAUSAL
    layer_windows: Sequence[int] = field(default_factory=tuple)
    device: int = 0
    shard_mode: int = SHARD_NONE
    shard_pos_begin: int = 0
    shard_pos_count: int = 0
    n_ranks: int = 1
    rank: int = 0
    decode_impl: int = IMPL_AUTO
    prefill_impl: int = IMPL_AUTO
    max_splits: int = 0
    decode_fusion: int = 0
    exchange_wait_us: int = 0

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def to_c(self):
        c = _Config()
        c.struct_size = C.sizeof(_Config)
        for name in ("n_layers", "n_heads", "n_kv_heads", "head_dim", "rope_dim", "seq_len", "max_batch",
                     "rope_theta", "rope_theta_swa", "rope_scale_global", "rope_scale_local", "rope_style",
                     "rope_layout", "swa_theta_on_window_layers", "swa_pattern", "scale_mode", "softmax_mode",
                     "kv_format", "image_mode", "device", "shard_mode", "shard_pos_begin", "shard_pos_count",
                     "n_ranks", "rank", "decode_impl", "prefill_impl", "max_splits", "decode_fusion",
                     "exchange_wait_us"):
            setattr(c, name, getattr(self, name))
        for i in range(4):
            c.rope_sections[i] = int(self.rope_sections[i])
        windows = (C.c_int32 * max(1, len(self.layer_windows)))(*[int(w) for w in self.layer_windows])
        c.n_layer_windows = len(self.layer_windows)
        c.layer_windows = C.cast(windows, C.POINTER(C.c_int32))
        return c, windows


class Weights:
    """One projection matrix [rows][cols] resident on a device, uploaded from the GGML row layout the reference maps
    from the GGUF file (F32, BF16, Q8_0 blocks of one f16 scale and 32 int8 codes, Q4_K super-blocks of 144 bytes or
    Q6_K super-blocks of 210 bytes per 256 weights)."""

    def __init__(self, wtype: int, rows: int, cols: int, data: np.ndarray, device: int = 0):
        self._L = lib()
        data = np.ascontiguousarray(data)
        want = {W_F32: rows * cols * 4, W_BF16: rows * cols * 2, W_Q8_0: rows * (cols // 32) * 34,
                W_Q4_K: rows * (cols // 256) * 144, W_Q6_K: rows * (cols // 256) * 210}.get(wtype, -1)
        if data.nbytes != want:
            raise ValueError(f"weight data has {data.nbytes} bytes, the layout needs {want}")
        h = C.c_void_p()
        st = self._L.ggr_weights_upload(device, wtype, rows, cols, C.c_void_p(data.ctypes.data), C.byref(h))
        if st != 0:
            raise GgrError(st, self._L.ggr_attn_create_error().decode())
        self._h, self.wtype, self.rows, self.cols = h, wtype, rows, cols

    def close(self):
        if getattr(self, "_h", None):
            self._L.ggr_weights_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RawCuda:
    """Lets torch view device memory owned by the library (__cuda_array_interface__), e.g. the cache arrays
    returned by AttnContext.kv_device_ptrs()."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _ptr(x, want_dtype=None):
    """(address, ptr_kind) of a numpy array or a torch tensor; checks contiguity."""
    if x is None:
        return None, None
    if _is_torch(x):
        if not x.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return C.c_void_p(x.data_ptr()), (PTR_DEVICE if x.is_cuda else PTR_HOST)
    a = x
    if not isinstance(a, np.ndarray) or not a.flags["C_CONTIGUOUS"]:
        raise ValueError("buffer must be a C-contiguous numpy array or a torch tensor")
    if want_dtype is not None and a.dtype != want_dtype:
        raise ValueError(f"buffer dtype {a.dtype} != {want_dtype}")
    return C.c_void_p(a.ctypes.data), PTR_HOST


class AttnContext:
    """One device KV cache + RoPE state; the KV half of the reference's RunState
    (malloc_run_state_with_kv_cache_format, src/engine/runtime/inference.rs:1529)."""

    def __init__(self, config: AttnConfig):
        self.config = config
        self._L = lib()
        c, keep = config.to_c()
        self._keep = keep
        handle = C.c_void_p()
        st = self._L.ggr_attn_create(C.byref(c), C.byref(handle))
        if st != 0:
            raise GgrError(st, self._L.ggr_attn_create_error().decode())
        self._h = handle
        self._stream = None

    def _follow_torch_stream(self, *tensors):
        """Device-pointer calls are enqueued on torch's current stream, so they are
        ordered with the kernels that produced the tensors and those that read the result."""
        for t in tensors:
            if t is not None and _is_torch(t) and t.is_cuda:
                import torch
                handle = torch.cuda.current_stream(t.device).cuda_stream or 1  # 0 is the legacy default stream
                if handle != self._stream:
                    self.set_stream(handle)
                return

    def close(self):
        if getattr(self, "_h", None):
            self._L.ggr_attn_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, st: int):
        if st != 0:
            raise GgrError(st, self._L.ggr_attn_last_error(self._h).decode())

    # ---- state -------------------------------------------------------------------------
    def set_stream(self, cuda_stream: int):
        """cuda_stream: a cudaStream_t value; 0 selects the stream the context owns,
        1 (cudaStreamLegacy) the legacy default stream."""
        self._check(self._L.ggr_attn_set_stream(self._h, C.c_void_p(cuda_stream)))
        self._stream = cuda_stream

    def synchronize(self):
        self._check(self._L.ggr_attn_synchronize(self._h))

    def set_position_plan(self, plan: Optional["RopePositionPlan"]):
        if plan is None:
            self._check(self._L.ggr_attn_set_position_plan(self._h, None, 0, 0))
            return
        rows = plan.export()
        self._check(self._L.ggr_attn_set_position_plan(
            self._h, C.c_void_p(rows.ctypes.data), rows.shape[0], plan.next_text_position))

    def set_media_blocks(self, blocks: Sequence[Sequence[int]], prompt_tokens: int):
        arr = np.ascontiguousarray(np.array(list(blocks), dtype=np.int32).reshape(-1, 2))
        self._check(self._L.ggr_attn_set_media_blocks(self._h, C.c_void_p(arr.ctypes.data), arr.shape[0],
                                                       prompt_tokens))

    def set_layer_fixups(self, layer: int, q_bias=None, k_bias=None, v_bias=None, q_norm=None, k_norm=None,
                         eps: float = 1e-6):
        """Qwen2 biases and per-head RMS QK-norm weights of one layer (qkv_bias_and_norm,
        src/engine/runtime/inference.rs:2535-2572); None clears."""
        arrs = [None if a is None else np.ascontiguousarray(a, dtype=np.float32)
                for a in (q_bias, k_bias, v_bias, q_norm, k_norm)]
        ptrs = [None if a is None else C.c_void_p(a.ctypes.data) for a in arrs]
        self._check(self._L.ggr_attn_set_layer_fixups(self._h, layer, *ptrs, eps))

    def visible_keys(self, layer: int, pos: int) -> range:
        s, e = C.c_int32(), C.c_int32()
        self._check(self._L.ggr_attn_visible_keys(self._h, layer, pos, C.byref(s), C.byref(e)))
        return range(s.value, e.value)

    @property
    def launch_count(self) -> int:
        return int(self._L.ggr_attn_launch_count(self._h))

    @property
    def last_split_count(self) -> int:
        return int(self._L.ggr_attn_last_split_count(self._h))

    def set_kernel_timing(self, enable: bool):
        self._check(self._L.ggr_attn_set_kernel_timing(self._h, 1 if enable else 0))

    def kernel_time(self, kind: int = 0, reset: bool = True):
        """(summed device milliseconds, launches) of one kernel kind: 0 attention, 1 rope/append, 2 merge."""
        ms, n = C.c_double(), C.c_int64()
        self._check(self._L.ggr_attn_kernel_time(self._h, kind, C.byref(ms), C.byref(n), 1 if reset else 0))
        return ms.value, n.value

    def kv_device_ptrs(self):
        """Device addresses (k, v, k_scale, v_scale) and the byte size of the K (or V) array."""
        k, v, ks, vs, nb = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_uint64()
        self._check(self._L.ggr_attn_kv_device_ptrs(self._h, C.byref(k), C.byref(v), C.byref(ks), C.byref(vs),
                                                     C.byref(nb)))
        return k.value, v.value, ks.value, vs.value, nb.value

    # ---- compute -----------------------------------------------------------------------
    def _out_like(self, q, shape):
        if _is_torch(q):
            import torch
            return torch.empty(shape, dtype=torch.float32, device=q.device)
        return np.empty(shape, dtype=np.float32)

    def decode(self, layer: int, pos, q, k, v, out=None):
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        B = pos.shape[0]
        if out is None:
            out = self._out_like(q, (B, self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (op, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(out)
        self._check(self._L.ggr_attn_decode(self._h, layer, C.c_void_p(pos.ctypes.data), B, qp, kp, vp, op, kind))
        return out

    def decode_gated(self, layer: int, pos, q, k, v, gate, gate_head_stride: Optional[int] = None, out=None):
        """decode followed by out *= sigmoid(gate), non-finite -> 0 (src/engine/runtime/inference.rs:3509-3519);
        gate is f32, head h of batch entry b at gate[(b * n_heads + h) * gate_head_stride]."""
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        B = pos.shape[0]
        if out is None:
            out = self._out_like(q, (B, self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (gp, _), (op, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(gate), _ptr(out)
        self._check(self._L.ggr_attn_decode_gated(self._h, layer, C.c_void_p(pos.ctypes.data), B, qp, kp, vp, gp,
                                                   gate_head_stride or self.config.head_dim, op, kind))
        return out

    def proj_matmul(self, w: "Weights", x, out=None):
        """out [n][w.rows] = x [n][w.cols] W^T (matmul_quantized_with_scratch, src/engine/kernels/quant.rs:7225)."""
        n = x.shape[0]
        if out is None:
            out = self._out_like(x, (n, w.rows))
        self._follow_torch_stream(x)
        (xp, kind), (op, _) = _ptr(x), _ptr(out)
        self._check(self._L.ggr_proj_matmul(self._h, w._h, xp, n, op, kind))
        return out

    def layer_decode(self, layer: int, pos, xb, wq, wk, wv, wo, out=None):
        """q/k/v projections, rope + append + attention, output projection for one token per sequence."""
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        if out is None:
            out = self._out_like(xb, (pos.shape[0], wo.rows))
        self._follow_torch_stream(xb)
        (xp, kind), (op, _) = _ptr(xb), _ptr(out)
        self._check(self._L.ggr_attn_layer_decode(self._h, layer, C.c_void_p(pos.ctypes.data), pos.shape[0], xp, wq._h,
                                                   wk._h, wv._h, wo._h, op, kind))
        return out

    def layer_prefill(self, layer: int, base_pos: int, xb, wq, wk, wv, wo, seq: int = 0, out=None):
        m = xb.shape[0]
        if out is None:
            out = self._out_like(xb, (m, wo.rows))
        self._follow_torch_stream(xb)
        (xp, kind), (op, _) = _ptr(xb), _ptr(out)
        self._check(self._L.ggr_attn_layer_prefill(self._h, layer, seq, base_pos, m, xp, wq._h, wk._h, wv._h, wo._h, op,
                                                    kind))
        return out

    def reserve(self, B: int):
        """Pre-allocates all decode scratch for batches of up to B sequences."""
        self._check(self._L.ggr_attn_reserve(self._h, B))

    def decode_partial(self, layer: int, pos, q, k, v, partial=None):
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        B = pos.shape[0]
        if partial is None:
            partial = self._out_like(q, (B, self.config.n_heads, self.config.head_dim + 2))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (pp, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(partial)
        self._check(self._L.ggr_attn_decode_partial(self._h, layer, C.c_void_p(pos.ctypes.data), B, qp, kp, vp, pp,
                                                     kind))
        return partial

    def exchange_create(self, max_B: int):
        """Allocates the local receive buffer of the fused shard exchange; returns (device address, 64-byte IPC handle)."""
        base = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        self._check(self._L.ggr_attn_exchange_create(self._h, max_B, C.byref(base), handle))
        return base.value, bytes(handle)

    def exchange_connect(self, ipc_handles=None, same_process_ptrs=None):
        """ipc_handles: list of n_ranks 64-byte handles (other processes); same_process_ptrs: list of device addresses."""
        hbuf = None
        if ipc_handles is not None:
            hbuf = (C.c_ubyte * (64 * len(ipc_handles)))(*b"".join(ipc_handles))
        pbuf = None
        if same_process_ptrs is not None:
            pbuf = (C.c_void_p * len(same_process_ptrs))(*[C.c_void_p(p) for p in same_process_ptrs])
        self._check(self._L.ggr_attn_exchange_connect(self._h, hbuf, pbuf))

    def decode_exchange(self, layer: int, pos, q, k, v, out=None):
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        B = pos.shape[0]
        if out is None:
            out = self._out_like(q, (B, self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (op, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(out)
        self._check(self._L.ggr_attn_decode_exchange(self._h, layer, C.c_void_p(pos.ctypes.data), B, qp, kp, vp, op, kind))
        return out

    def exchange_send(self, layer: int, pos, q, k, v):
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _) = _ptr(q), _ptr(k), _ptr(v)
        self._check(self._L.ggr_attn_exchange_send(self._h, layer, C.c_void_p(pos.ctypes.data), pos.shape[0], qp, kp, vp,
                                                    kind))

    @property
    def exchange_epoch(self) -> int:
        return int(self._L.ggr_attn_exchange_epoch(self._h))

    def exchange_resync(self, epoch: int):
        self._check(self._L.ggr_attn_exchange_resync(self._h, epoch))

    def exchange_receive(self, B: int, like, out=None):
        if out is None:
            out = self._out_like(like, (B, self.config.q_dim))
        self._follow_torch_stream(like)
        (op, kind) = _ptr(out)
        self._check(self._L.ggr_attn_exchange_receive(self._h, B, op, kind))
        return out

    def combine_partials(self, parts, out=None):
        n_parts, B = parts.shape[0], parts.shape[1]
        if out is None:
            out = self._out_like(parts, (B, self.config.q_dim))
        self._follow_torch_stream(parts)
        (pp, kind), (op, _) = _ptr(parts), _ptr(out)
        self._check(self._L.ggr_attn_combine_partials(self._h, pp, n_parts, B, op, kind))
        return out

    def _prefill(self, fn, layer, seq, base_pos, q, k, v, out):
        m = q.shape[0]
        if _is_torch(q):
            import torch
            in_dtype = DTYPE_BF16 if q.dtype == torch.bfloat16 else DTYPE_F32
        else:
            in_dtype = DTYPE_BF16 if q.dtype == np.uint16 else DTYPE_F32
        if out is None:
            out = self._out_like(q, (m, self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (op, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(out)
        self._check(fn(self._h, layer, seq, base_pos, m, qp, kp, vp, in_dtype, op, kind))
        return out

    def prefill(self, layer: int, base_pos: int, q, k, v, seq: int = 0, out=None):
        """q/k/v: [m, q_dim] / [m, kv_dim], f32, or bf16 (torch.bfloat16 / numpy uint16 bit patterns)."""
        return self._prefill(self._L.ggr_attn_prefill, layer, seq, base_pos, q, k, v, out)

    def prefill_gated(self, layer: int, base_pos: int, q, k, v, gate, gate_head_stride: Optional[int] = None,
                      seq: int = 0, out=None):
        """prefill with the output gate of decode_gated; gate has the dtype of q."""
        m = q.shape[0]
        if _is_torch(q):
            import torch
            in_dtype = DTYPE_BF16 if q.dtype == torch.bfloat16 else DTYPE_F32
        else:
            in_dtype = DTYPE_BF16 if q.dtype == np.uint16 else DTYPE_F32
        if out is None:
            out = self._out_like(q, (m, self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, kind), (kp, _), (vp, _), (gp, _), (op, _) = _ptr(q), _ptr(k), _ptr(v), _ptr(gate), _ptr(out)
        self._check(self._L.ggr_attn_prefill_gated(self._h, layer, seq, base_pos, m, qp, kp, vp, gp,
                                                    gate_head_stride or self.config.head_dim, in_dtype, op, kind))
        return out

    def prefill_block(self, layer: int, base_pos: int, q, k, v, seq: int = 0, out=None):
        return self._prefill(self._L.ggr_attn_prefill_block, layer, seq, base_pos, q, k, v, out)

    def apply_rope_qk(self, layer: int, pos: int, q, k):
        """Rotates q and k in place (apply_rope_qk, src/engine/runtime/inference.rs:1817)."""
        self._follow_torch_stream(q)
        (qp, kind), (kp, _) = _ptr(q), _ptr(k)
        self._check(self._L.ggr_attn_apply_rope_qk(self._h, layer, pos, qp, kp, kind))

    def kv_write_token(self, layer: int, pos: int, k, v, seq: int = 0):
        self._follow_torch_stream(k)
        (kp, kind), (vp, _) = _ptr(k), _ptr(v)
        self._check(self._L.ggr_attn_kv_write_token(self._h, seq, layer, pos, kp, vp, kind))

    def attention_token(self, layer: int, pos: int, q, seq: int = 0, out=None):
        if out is None:
            out = self._out_like(q, (self.config.q_dim,))
        self._follow_torch_stream(q)
        (qp, kind), (op, _) = _ptr(q), _ptr(out)
        self._check(self._L.ggr_attn_attention_token(self._h, seq, layer, pos, qp, op, kind))
        return out

    def attention_tokens_static(self, layer: int, pos, q, out=None):
        """Attention of B already rotated query rows (torch CUDA tensors) using the library's
        built-in scratch array: nothing is allocated by the call (see include/ggr_attn.h)."""
        pos = np.ascontiguousarray(np.asarray(pos, dtype=np.int32).reshape(-1))
        if not (_is_torch(q) and q.is_cuda):
            raise ValueError("attention_tokens_static takes device memory only")
        if out is None:
            out = self._out_like(q, (pos.shape[0], self.config.q_dim))
        self._follow_torch_stream(q)
        (qp, _), (op, _) = _ptr(q), _ptr(out)
        self._check(self._L.ggr_attn_attention_tokens_static(self._h, layer, C.c_void_p(pos.ctypes.data),
                                                              pos.shape[0], qp, op))
        return out

    # ---- cache access ------------------------------------------------------------------
    def kv_read_row(self, layer: int, pos: int, seq: int = 0):
        k = np.empty(self.config.kv_dim, dtype=np.float32)
        v = np.empty(self.config.kv_dim, dtype=np.float32)
        self._check(self._L.ggr_attn_kv_read_row(self._h, seq, layer, pos, C.c_void_p(k.ctypes.data),
                                                  C.c_void_p(v.ctypes.data)))
        return k, v

    def kv_read_turbo(self, layer: int, pos: int, seq: int = 0):
        """Raw TurboQuant row (src/engine/runtime/inference.rs:1919-1963): codes, sign bits, sigma and residual norm."""
        kd, H = self.config.kv_dim, self.config.n_kv_heads
        out = {"k_base": np.empty(kd // 4, np.uint8), "v_base": np.empty(kd // 4, np.uint8),
               "k_sign": np.empty(kd // 8, np.uint8), "v_sign": np.empty(kd // 8, np.uint8),
               "k_scale": np.empty(H, np.float32), "v_scale": np.empty(H, np.float32),
               "k_rnorm": np.empty(H, np.float32), "v_rnorm": np.empty(H, np.float32)}
        order = ("k_base", "v_base", "k_sign", "v_sign", "k_scale", "v_scale", "k_rnorm", "v_rnorm")
        self._check(self._L.ggr_attn_kv_read_turbo(self._h, seq, layer, pos,
                                                    *[C.c_void_p(out[n].ctypes.data) for n in order]))
        return out

    def kv_export(self, layer: int, row0: int, nrows: int, seq: int = 0):
        kd = self.config.kv_dim
        kq = np.empty((nrows, kd), dtype=np.int8)
        vq = np.empty((nrows, kd), dtype=np.int8)
        scale_shape = (nrows,) if self.config.kv_format == KV_Q8_ROW else (nrows, kd // 32)
        ks = np.empty(scale_shape, dtype=np.float32)
        vs = np.empty(scale_shape, dtype=np.float32)
        self._check(self._L.ggr_attn_kv_export(self._h, layer, seq, row0, nrows, C.c_void_p(kq.ctypes.data),
                                                C.c_void_p(vq.ctypes.data), C.c_void_p(ks.ctypes.data),
                                                C.c_void_p(vs.ctypes.data)))
        return kq, vq, ks, vs

    def kv_import(self, layer: int, row0: int, kq, vq, ks, vs, seq: int = 0):
        kq = np.ascontiguousarray(kq, dtype=np.int8)
        vq = np.ascontiguousarray(vq, dtype=np.int8)
        ks = np.ascontiguousarray(ks, dtype=np.float32)
        vs = np.ascontiguousarray(vs, dtype=np.float32)
        self._check(self._L.ggr_attn_kv_import(self._h, layer, seq, row0, kq.shape[0], C.c_void_p(kq.ctypes.data),
                                                C.c_void_p(vq.ctypes.data), C.c_void_p(ks.ctypes.data),
                                                C.c_void_p(vs.ctypes.data)))


    _TURBO_SECTIONS = ("k_base", "v_base", "k_sign", "v_sign", "k_scale", "v_scale", "k_rnorm", "v_rnorm")

    def kv_export_turbo(self, layer: int, row0: int, nrows: int, seq: int = 0):
        """Rows of a TurboQuant cache as the eight sections of the reference's prefill cache
        (src/app/prefill_cache.rs:16-18)."""
        kd, H = self.config.kv_dim, self.config.n_kv_heads
        out = {"k_base": np.empty((nrows, kd // 4), np.uint8), "v_base": np.empty((nrows, kd // 4), np.uint8),
               "k_sign": np.empty((nrows, kd // 8), np.uint8), "v_sign": np.empty((nrows, kd // 8), np.uint8),
               "k_scale": np.empty((nrows, H), np.float32), "v_scale": np.empty((nrows, H), np.float32),
               "k_rnorm": np.empty((nrows, H), np.float32), "v_rnorm": np.empty((nrows, H), np.float32)}
        self._check(self._L.ggr_attn_kv_export_turbo(self._h, layer, seq, row0, nrows,
                                                      *[C.c_void_p(out[n].ctypes.data) for n in self._TURBO_SECTIONS]))
        return out

    def kv_import_turbo(self, layer: int, row0: int, sections, seq: int = 0):
        arrs = [np.ascontiguousarray(sections[n]) for n in self._TURBO_SECTIONS]
        self._check(self._L.ggr_attn_kv_import_turbo(self._h, layer, seq, row0, arrs[0].shape[0],
                                                      *[C.c_void_p(a.ctypes.data) for a in arrs]))


class RopePositionPlan:
    """Logical T/H/W coordinates per physical KV row (src/engine/positions.rs:3-54)."""

    def __init__(self):
        self._L = lib()
        self._h = C.c_void_p(self._L.ggr_rope_plan_new())

    def __del__(self):
        try:
            if self._h:
                self._L.ggr_rope_plan_free(self._h)
                self._h = None
        except Exception:
            pass

    def append_text(self, count: int):
        if self._L.ggr_rope_plan_append_text(self._h, count) != 0:
            raise ValueError("text rotary position overflow")

    def append_grid(self, grid: Sequence[int], token_count: int):
        t, h, w = grid
        if min(t, h, w) < 0 or max(t, h, w, token_count) >= 2 ** 63:
            raise ValueError("image rotary grid size overflow")
        if self._L.ggr_rope_plan_append_grid(self._h, t, h, w, token_count) != 0:
            raise ValueError(f"image rotary grid {list(grid)} does not hold {token_count} embeddings")

    def __len__(self) -> int:
        return int(self._L.ggr_rope_plan_len(self._h))

    @property
    def next_text_position(self) -> int:
        return int(self._L.ggr_rope_plan_next_text(self._h))

    def at(self, pos: int):
        out = (C.c_int64 * 3)()
        self._L.ggr_rope_plan_at(self._h, pos, out)
        return [int(out[0]), int(out[1]), int(out[2])]

    def export(self) -> np.ndarray:
        n = len(self)
        rows = np.zeros((max(n, 1), 3), dtype=np.int32)
        self._L.ggr_rope_plan_export(self._h, C.c_void_p(rows.ctypes.data), n)
        return rows[:n]

    @property
    def positions(self):
        return self.export().tolist()


class MediaAttentionPlan:
    """Validated image blocks (src/engine/runtime/attention.rs:8-70)."""

    def __init__(self, prompt_tokens: int, blocks: Sequence[Sequence[int]]):
        self._L = lib()
        self.prompt_tokens = prompt_tokens
        self.blocks = [(int(s), int(n)) for s, n in blocks]
        for s, n in self.blocks:
            if not (0 <= s < 2 ** 63 and 0 <= n < 2 ** 63):
                raise ValueError("image attention block range overflow")
        self._arr = np.ascontiguousarray(np.array(self.blocks, dtype=np.int64).reshape(-1, 2))
        if self._L.ggr_media_plan_validate(C.c_void_p(self._arr.ctypes.data), len(self.blocks), prompt_tokens) != 0:
            raise ValueError("image attention blocks must be nonempty, ordered, disjoint, and within the prompt")

    def block_at(self, position: int):
        for s, n in self.blocks:
            if s <= position < s + n:
                return (s, n)
        return None

    def chunk_end(self, start: int, limit: int, chunk: int) -> int:
        chunk = min(chunk, 2 ** 63 - 1)
        r = self._L.ggr_media_chunk_end(C.c_void_p(self._arr.ctypes.data), len(self.blocks), self.prompt_tokens,
                                        start, limit, chunk)
        if r < 0:
            raise ValueError("invalid media prefill chunk")
        return int(r)


def rope_axis(layout: int, frequency: int, sections: Sequence[int]) -> int:
    sec = (C.c_int32 * 4)(*[int(s) for s in sections])
    return int(lib().ggr_rope_axis(layout, frequency, sec))


def gemma_layer_windows(n_layers: int, window: int, period: int = 6):
    out = np.zeros(max(n_layers, 1), dtype=np.int32)
    if lib().ggr_gemma_layer_windows(n_layers, window, period, C.c_void_p(out.ctypes.data)) != 0:
        raise ValueError("invalid window pattern")
    return out[:n_layers].tolist()
