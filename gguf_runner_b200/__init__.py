"""B200 (sm_100a) attention path for gguf-runner: Python mirror of the C ABI.

The product is `libggr_attn.so` (hand-written CUDA kernels behind the C ABI in
`include/ggr_attn.h`). This package only binds it with ctypes so tests and the
benchmark can drive the same entry points a Rust host would bind through FFI.
There is no fallback: if the library is missing or no CUDA device exists, the
calls raise.
"""
from .binding import (  # noqa: F401
    AttnConfig,
    AttnContext,
    GgrError,
    MediaAttentionPlan,
    RopePositionPlan,
    Weights,
    gemma_layer_windows,
    lib,
    library_path,
    rope_axis,
)
from . import presets  # noqa: F401
from . import sharding  # noqa: F401
