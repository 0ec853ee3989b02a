"""ctypes access to the CPU oracle (oracle/libggr_oracle.so) for tests, the
smoke check and the benchmark's CPU-baseline leg. Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_LIB = None


class OraConfig(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("rope_dim", C.c_int32), ("seq_len", C.c_int32), ("max_batch", C.c_int32),
        ("rope_theta", C.c_float), ("rope_theta_swa", C.c_float),
        ("rope_scale_global", C.c_float), ("rope_scale_local", C.c_float),
        ("rope_style", C.c_int32), ("rope_layout", C.c_int32), ("rope_sections", C.c_int32 * 4),
        ("swa_theta_on_window_layers", C.c_int32), ("swa_pattern", C.c_int32),
        ("scale_mode", C.c_int32), ("softmax_mode", C.c_int32), ("kv_format", C.c_int32),
        ("image_mode", C.c_int32), ("n_layer_windows", C.c_int32),
        ("layer_windows", C.POINTER(C.c_int32)),
    ]


def build(force: bool = False) -> str:
    path = os.path.join(ORACLE_DIR, "libggr_oracle.so")
    src = [os.path.join(ORACLE_DIR, f) for f in ("ref_attention.cpp", "ref_attention.h", "Makefile")]
    stale = (not os.path.exists(path)) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in src)
    if force or stale:
        subprocess.run(["make", "-C", ORACLE_DIR, "-B"], check=True, capture_output=True)
    return path


def build_native() -> str:
    """The same source compiled for the host it runs on (-O3 -march=native), for the CPU-baseline timing legs
    only: it is built where it is used (a library built for one CPU may not run on another) and never checked
    against golden vectors; parity always uses the strict build above."""
    out_dir = os.path.join(ORACLE_DIR, "_native")
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "libggr_oracle_native.so")
    src = os.path.join(ORACLE_DIR, "ref_attention.cpp")
    if not os.path.exists(path) or os.path.getmtime(src) > os.path.getmtime(path):
        subprocess.run([os.environ.get("CXX", "g++"), "-O3", "-march=native", "-ffp-contract=off", "-fno-fast-math",
                        "-funroll-loops", "-fPIC", "-std=c++17", "-pthread", "-shared", "-o", path, src],
                       check=True, capture_output=True)
    return path


_NATIVE = None


def lib(native: bool = False) -> C.CDLL:
    global _LIB, _NATIVE
    if native:
        if _NATIVE is None:
            _NATIVE = _bind(C.CDLL(build_native()))
        return _NATIVE
    if _LIB is not None:
        return _LIB
    _LIB = _bind(C.CDLL(build()))
    return _LIB


def _bind(L: C.CDLL) -> C.CDLL:
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    L.ora_create.argtypes = [C.POINTER(OraConfig), C.POINTER(vp), C.POINTER(C.c_char_p)]
    L.ora_destroy.argtypes = [vp]
    L.ora_destroy.restype = None
    L.ora_set_threads.argtypes = [vp, C.c_int]
    L.ora_set_threads.restype = None
    L.ora_set_position_plan.argtypes = [vp, vp, i32, i32]
    L.ora_set_media_blocks.argtypes = [vp, vp, i32, i32]
    L.ora_set_layer_fixups.argtypes = [vp, i32, vp, vp, vp, vp, vp, C.c_float]
    L.ora_qkv_bias_and_norm.argtypes = [vp, i32, vp, vp, vp]
    L.ora_qkv_bias_and_norm.restype = None
    L.ora_matmul.argtypes = [i32, i32, i32, vp, vp, vp]
    L.ora_matmul.restype = None
    L.ora_fp16_to_fp32.argtypes = [C.c_uint16]
    L.ora_fp16_to_fp32.restype = C.c_float
    L.ora_sigmoid_gate.argtypes = [vp, vp, vp, i32]
    L.ora_sigmoid_gate.restype = None
    L.ora_rope_angles.argtypes = [vp, i32, i32, vp, vp]
    L.ora_rope_angles.restype = None
    L.ora_apply_rope_qk.argtypes = [vp, i32, i32, vp, vp]
    L.ora_apply_rope_qk.restype = None
    L.ora_kv_write_token.argtypes = [vp, i32, i32, i32, vp, vp]
    L.ora_kv_write_token.restype = None
    L.ora_attention_token.argtypes = [vp, i32, i32, i32, vp, vp]
    L.ora_attention_token.restype = None
    L.ora_visible_keys.argtypes = [vp, i32, i32, C.POINTER(i32), C.POINTER(i32)]
    L.ora_visible_keys.restype = None
    L.ora_decode.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp]
    L.ora_decode.restype = None
    L.ora_prefill.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.ora_prefill.restype = None
    L.ora_prefill_block.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.ora_prefill_block.restype = None
    L.ora_kv_read_row.argtypes = [vp, i32, i32, i32, vp, vp]
    L.ora_kv_read_row.restype = None
    L.ora_kv_read_q8.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp]
    L.ora_kv_read_turbo.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]
    L.ora_kv_read_turbo.restype = C.c_int
    L.ora_turbo_transform.argtypes = [vp, i32, i32, i32, i32, vp]
    L.ora_turbo_transform.restype = C.c_int
    L.ora_plan_new.restype = vp
    L.ora_plan_free.argtypes = [vp]
    L.ora_plan_free.restype = None
    L.ora_plan_append_text.argtypes = [vp, i64]
    L.ora_plan_append_grid.argtypes = [vp, i64, i64, i64, i64]
    L.ora_plan_len.argtypes = [vp]
    L.ora_plan_len.restype = i64
    L.ora_plan_next_text.argtypes = [vp]
    L.ora_plan_next_text.restype = i64
    L.ora_plan_at.argtypes = [vp, i64, C.POINTER(i64)]
    L.ora_plan_at.restype = None
    L.ora_rope_axis.argtypes = [i32, i32, C.POINTER(i32)]
    L.ora_media_plan_validate.argtypes = [vp, i32, i64]
    L.ora_media_chunk_end.argtypes = [vp, i32, i64, i64, i64, i64]
    L.ora_media_chunk_end.restype = i64
    L.ora_gemma_layer_windows.argtypes = [i32, i32, i32, vp]
    L.ora_f32_to_bf16.argtypes = [C.c_float]
    L.ora_f32_to_bf16.restype = C.c_uint16
    L.ora_bf16_to_f32.argtypes = [C.c_uint16]
    L.ora_bf16_to_f32.restype = C.c_float
    return L


def _p(a):
    return C.c_void_p(a.ctypes.data)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class OraclePlan:
    def __init__(self):
        self.L = lib()
        self.h = C.c_void_p(self.L.ora_plan_new())

    def __del__(self):
        if getattr(self, "h", None):
            self.L.ora_plan_free(self.h)
            self.h = None

    def append_text(self, n):
        return self.L.ora_plan_append_text(self.h, n)

    def append_grid(self, grid, count):
        return self.L.ora_plan_append_grid(self.h, grid[0], grid[1], grid[2], count)

    def __len__(self):
        return int(self.L.ora_plan_len(self.h))

    @property
    def next_text_position(self):
        return int(self.L.ora_plan_next_text(self.h))

    def at(self, pos):
        out = (C.c_int64 * 3)()
        self.L.ora_plan_at(self.h, pos, out)
        return [int(x) for x in out]

    @property
    def positions(self):
        return [self.at(i) for i in range(len(self))]


class Oracle:
    """CPU restatement of the reference attention path, configured from the same
    fields as gguf_runner_b200.AttnConfig (any object with those attributes)."""

    def __init__(self, cfg, threads: int = 1, native: bool = False):
        self.L = lib(native)
        self.cfg = cfg
        c = OraConfig()
        for name in ("n_layers", "n_heads", "n_kv_heads", "head_dim", "rope_dim", "seq_len", "max_batch",
                     "rope_theta", "rope_theta_swa", "rope_scale_global", "rope_scale_local", "rope_style",
                     "rope_layout", "swa_theta_on_window_layers", "swa_pattern", "scale_mode", "softmax_mode",
                     "kv_format", "image_mode"):
            setattr(c, name, getattr(cfg, name))
        for i in range(4):
            c.rope_sections[i] = int(cfg.rope_sections[i])
        w = list(cfg.layer_windows)
        self._w = (C.c_int32 * max(1, len(w)))(*w)
        c.n_layer_windows = len(w)
        c.layer_windows = C.cast(self._w, C.POINTER(C.c_int32))
        h = C.c_void_p()
        err = C.c_char_p()
        st = self.L.ora_create(C.byref(c), C.byref(h), C.byref(err))
        if st != 0:
            raise ValueError(err.value.decode() if err.value else f"oracle status {st}")
        self.h = h
        self.q_dim = cfg.n_heads * cfg.head_dim
        self.kv_dim = cfg.n_kv_heads * cfg.head_dim
        self.L.ora_set_threads(self.h, threads)

    def close(self):
        if getattr(self, "h", None):
            self.L.ora_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def set_threads(self, n):
        self.L.ora_set_threads(self.h, n)

    def set_position_plan(self, rows, next_text):
        rows = np.ascontiguousarray(np.asarray(rows, dtype=np.int32).reshape(-1, 3))
        self.L.ora_set_position_plan(self.h, _p(rows), rows.shape[0], next_text)

    def set_media_blocks(self, blocks, prompt_tokens):
        arr = np.ascontiguousarray(np.asarray(blocks, dtype=np.int32).reshape(-1, 2))
        if self.L.ora_set_media_blocks(self.h, _p(arr), arr.shape[0], prompt_tokens) != 0:
            raise ValueError("invalid blocks")

    def set_layer_fixups(self, layer, q_bias=None, k_bias=None, v_bias=None, q_norm=None, k_norm=None, eps=1e-6):
        arrs = [None if a is None else _f32(a) for a in (q_bias, k_bias, v_bias, q_norm, k_norm)]
        self._fix = arrs
        ptrs = [None if a is None else _p(a) for a in arrs]
        if self.L.ora_set_layer_fixups(self.h, layer, *ptrs, eps) != 0:
            raise ValueError("bad layer")

    def rope_angles(self, layer, pos):
        half = (self.cfg.rope_dim or self.cfg.head_dim) // 2
        c = np.empty(half, np.float32)
        s = np.empty(half, np.float32)
        self.L.ora_rope_angles(self.h, layer, pos, _p(c), _p(s))
        return c, s

    def apply_rope_qk(self, layer, pos, q, k):
        self.L.ora_apply_rope_qk(self.h, layer, pos, _p(q), _p(k))

    def kv_write_token(self, layer, pos, k, v, seq=0):
        k, v = _f32(k), _f32(v)
        self.L.ora_kv_write_token(self.h, seq, layer, pos, _p(k), _p(v))

    def attention_token(self, layer, pos, q, seq=0):
        q = _f32(q)
        out = np.empty(self.q_dim, np.float32)
        self.L.ora_attention_token(self.h, seq, layer, pos, _p(q), _p(out))
        return out

    def visible_keys(self, layer, pos):
        s, e = C.c_int32(), C.c_int32()
        self.L.ora_visible_keys(self.h, layer, pos, C.byref(s), C.byref(e))
        return range(s.value, e.value)

    def decode(self, layer, pos, q, k, v):
        pos = np.ascontiguousarray(np.asarray(pos, np.int32).reshape(-1))
        q, k, v = _f32(q), _f32(k), _f32(v)
        out = np.empty((pos.shape[0], self.q_dim), np.float32)
        self.L.ora_decode(self.h, layer, _p(pos), pos.shape[0], _p(q), _p(k), _p(v), _p(out))
        return out

    def sigmoid_gate(self, out, gate, gate_head_stride=None):
        """Applies the output gate in place to rows of attention output [n][q_dim]; gate rows hold
        n_heads heads at a stride of gate_head_stride elements (default head_dim)."""
        stride = gate_head_stride or self.cfg.head_dim
        gate = _f32(gate)
        row = self.cfg.n_heads * stride
        for i in range(out.shape[0]):
            g = gate.reshape(-1)[i * row:]
            self.L.ora_sigmoid_gate(self.h, C.c_void_p(out[i].ctypes.data), C.c_void_p(g.ctypes.data), stride)
        return out

    def prefill(self, layer, base_pos, q, k, v, seq=0, block=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        m = q.shape[0]
        out = np.empty((m, self.q_dim), np.float32)
        fn = self.L.ora_prefill_block if block else self.L.ora_prefill
        fn(self.h, layer, seq, base_pos, m, _p(q), _p(k), _p(v), _p(out))
        return out

    def kv_read_row(self, layer, pos, seq=0):
        k = np.empty(self.kv_dim, np.float32)
        v = np.empty(self.kv_dim, np.float32)
        self.L.ora_kv_read_row(self.h, seq, layer, pos, _p(k), _p(v))
        return k, v

    def kv_read_q8(self, layer, pos, seq=0):
        kq = np.empty(self.kv_dim, np.int8)
        vq = np.empty(self.kv_dim, np.int8)
        ns = 1 if self.cfg.kv_format == 2 else self.kv_dim // 32
        ks = np.empty(ns, np.float32)
        vs = np.empty(ns, np.float32)
        if self.L.ora_kv_read_q8(self.h, seq, layer, pos, _p(kq), _p(vq), _p(ks), _p(vs)) != 0:
            raise ValueError("not a q8 cache")
        return kq, vq, ks, vs

    def kv_read_turbo(self, layer, pos, seq=0):
        """Raw TurboQuant row: dict of codes, sign bits and the per-head sigma / residual norm of K and V."""
        kd, H = self.kv_dim, self.cfg.n_kv_heads
        out = {"k_base": np.empty(kd // 4, np.uint8), "v_base": np.empty(kd // 4, np.uint8),
               "k_sign": np.empty(kd // 8, np.uint8), "v_sign": np.empty(kd // 8, np.uint8),
               "k_scale": np.empty(H, np.float32), "v_scale": np.empty(H, np.float32),
               "k_rnorm": np.empty(H, np.float32), "v_rnorm": np.empty(H, np.float32)}
        order = ("k_base", "v_base", "k_sign", "v_sign", "k_scale", "v_scale", "k_rnorm", "v_rnorm")
        if self.L.ora_kv_read_turbo(self.h, seq, layer, pos, *[_p(out[n]) for n in order]) != 0:
            raise ValueError("not a TurboQuant cache")
        return out

    def turbo_transform(self, layer, kv_head, first_slot, second_slot, values):
        v = np.ascontiguousarray(values, dtype=np.float32).copy()
        if self.L.ora_turbo_transform(self.h, layer, kv_head, first_slot, second_slot, _p(v)) != 0:
            raise ValueError("not a TurboQuant cache")
        return v


def matmul(wtype: int, rows: int, cols: int, w_raw: np.ndarray, x: np.ndarray) -> np.ndarray:
    """Reference matmul of every row of x [n][cols] with W (raw GGML bytes): returns [n][rows]."""
    x = _f32(x).reshape(-1, cols)
    w_raw = np.ascontiguousarray(w_raw)
    out = np.empty((x.shape[0], rows), np.float32)
    for i in range(x.shape[0]):
        lib().ora_matmul(wtype, rows, cols, _p(w_raw), _p(x[i]), C.c_void_p(out[i].ctypes.data))
    return out


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """GGML Q8_0 bytes of a float matrix [rows][cols] (cols % 32 == 0): per block of 32 one f16 scale
    d = max|w| / 127 and the codes round(w / d). Test helper: the reference only reads this layout."""
    rows, cols = w.shape
    blocks = w.reshape(rows, cols // 32, 32).astype(np.float32)
    d = (np.abs(blocks).max(axis=2) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1.0), 0.0)
    q = np.clip(np.rint(blocks * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((rows, cols // 32, 34), np.uint8)
    out[..., :2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """GGML Q4_K bytes of a float matrix [rows][cols] (cols % 256 == 0): super-blocks of 256 weights = f16 d,
    f16 dmin, eight 6-bit (scale, min) pairs packed into 12 bytes the way get_scale_min_k4 reads them
    (src/engine/kernels/quant.rs:118-126) and 128 bytes of nibbles (groups of 64: low nibbles, then high nibbles;
    dequantize_row_q4_k :294-325). w ~ d * scale * q - dmin * min. Test helper: a simple min / max quantiser, the
    reference only reads this layout."""
    rows, cols = w.shape
    nsb = cols // 256
    x = w.reshape(rows, nsb, 8, 32).astype(np.float32)
    lo = np.minimum(x.min(axis=3), 0.0)
    hi = np.maximum(x.max(axis=3), lo + 1e-12)
    step = (hi - lo) / 15.0                      # per 32 weights
    off = -lo                                    # >= 0
    d = (step.max(axis=2) / 63.0).astype(np.float16)
    dmin = (off.max(axis=2) / 63.0).astype(np.float16)
    df, mf = d.astype(np.float32)[..., None], dmin.astype(np.float32)[..., None]
    s6 = np.clip(np.rint(np.where(df > 0, step / np.where(df > 0, df, 1.0), 0.0)), 0, 63).astype(np.uint8)
    m6 = np.clip(np.rint(np.where(mf > 0, off / np.where(mf > 0, mf, 1.0), 0.0)), 0, 63).astype(np.uint8)
    eff = df * s6.astype(np.float32)
    q = np.where(eff[..., None] > 0, (x + (mf * m6.astype(np.float32))[..., None]) / np.where(eff > 0, eff, 1.0)[..., None], 0.0)
    q = np.clip(np.rint(q), 0, 15).astype(np.uint8)          # [rows][nsb][8][32]
    out = np.zeros((rows, nsb, 144), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nsb, 2)
    out[..., 2:4] = dmin.view(np.uint8).reshape(rows, nsb, 2)
    for j in range(4):
        out[..., 4 + j] = s6[..., j] | ((s6[..., j + 4] >> 4) << 6)
        out[..., 8 + j] = m6[..., j] | ((m6[..., j + 4] >> 4) << 6)
        out[..., 12 + j] = (s6[..., j + 4] & 0x0F) | ((m6[..., j + 4] & 0x0F) << 4)
    for grp in range(4):
        out[..., 16 + 32 * grp:16 + 32 * (grp + 1)] = q[:, :, 2 * grp, :] | (q[:, :, 2 * grp + 1, :] << 4)
    return out.reshape(rows, -1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    """GGML Q6_K bytes of a float matrix [rows][cols] (cols % 256 == 0): super-blocks of 256 weights = 128 bytes of
    low nibbles, 64 bytes of high bit pairs, 16 int8 scales (one per 16 weights) and an f16 d, laid out the way
    dequantize_row_q6_k reads them (src/engine/kernels/quant.rs:484-517): w ~ d * scale * (q - 32), q in 0..63.
    Test helper: a simple max-abs quantiser, the reference only reads this layout."""
    rows, cols = w.shape
    nsb = cols // 256
    x = w.reshape(rows, nsb, 16, 16).astype(np.float32)
    amax = np.abs(x).max(axis=3)                                  # per 16 weights
    d = (amax.max(axis=2) / 31.0 / 127.0).astype(np.float16)
    df = d.astype(np.float32)[..., None]
    sc = np.clip(np.rint(np.where(df > 0, amax / 31.0 / np.where(df > 0, df, 1.0), 0.0)), 1, 127).astype(np.int8)
    eff = df * sc.astype(np.float32)
    q = np.clip(np.rint(np.where(eff[..., None] > 0, x / np.where(eff > 0, eff, 1.0)[..., None], 0.0)), -32, 31).astype(np.int32) + 32
    q = q.reshape(rows, nsb, 2, 4, 32).astype(np.uint8)           # [half of 128][k: 32-weight run][l]
    out = np.zeros((rows, nsb, 210), np.uint8)
    for half in range(2):
        q1, q2, q3, q4 = (q[:, :, half, k, :] for k in range(4))
        out[..., 64 * half:64 * half + 32] = (q1 & 0x0F) | ((q3 & 0x0F) << 4)
        out[..., 64 * half + 32:64 * half + 64] = (q2 & 0x0F) | ((q4 & 0x0F) << 4)
        out[..., 128 + 32 * half:128 + 32 * half + 32] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    out[..., 192:208] = sc.view(np.uint8)
    out[..., 208:210] = d.view(np.uint8).reshape(rows, nsb, 2)
    return out.reshape(rows, -1)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as f32 (src/engine/io/gguf.rs:107-116)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) of an f32 array, round-to-nearest-even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16).reshape(a.shape)
