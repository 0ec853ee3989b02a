"""Attention settings the reference would configure for the benchmark's five
model shapes (family flags at src/vendors/mod.rs:711-862 and :906-1032,
Gemma window pattern at src/vendors/gemma.rs:63-105)."""
from __future__ import annotations

from .binding import (AttnConfig, IMAGE_BIDIRECTIONAL, KV_BF16, KV_F32, ROPE_ADJACENT, ROPE_NEOX,
                      SCALE_Q_PRESCALED, gemma_layer_windows)


def qwen3_0p6b_decode(n_layers=28, seq_len=2048, kv_format=KV_F32, **kw) -> AttnConfig:
    """Config 1: 16 query / 8 KV heads, head_dim 128, NeoX RoPE theta 1e6."""
    return AttnConfig(n_layers=n_layers, n_heads=16, n_kv_heads=8, head_dim=128, seq_len=seq_len,
                      rope_theta=1e6, rope_style=ROPE_NEOX, kv_format=kv_format, **kw)


def llama3_8b_prefill(n_layers=32, seq_len=4096, kv_format=KV_BF16, **kw) -> AttnConfig:
    """Config 2: 32 query / 8 KV heads, head_dim 128, adjacent-pair RoPE theta 5e5."""
    return AttnConfig(n_layers=n_layers, n_heads=32, n_kv_heads=8, head_dim=128, seq_len=seq_len,
                      rope_theta=5e5, rope_style=ROPE_ADJACENT, kv_format=kv_format, **kw)


def qwen3_30b_a3b_decode(n_layers=48, seq_len=32768, max_batch=1, kv_format=KV_BF16, **kw) -> AttnConfig:
    """Config 3: 32 query / 4 KV heads (GQA 8:1), head_dim 128, NeoX RoPE theta 1e6."""
    return AttnConfig(n_layers=n_layers, n_heads=32, n_kv_heads=4, head_dim=128, seq_len=seq_len,
                      max_batch=max_batch, rope_theta=1e6, rope_style=ROPE_NEOX, kv_format=kv_format, **kw)


def gemma3_4b_prefill(n_layers=34, seq_len=32768, window=1024, kv_format=KV_BF16, **kw) -> AttnConfig:
    """Config 4: 8 query / 4 KV heads, head_dim 256, five window layers to one global layer,
    theta 1e4 on window layers and 1e6 on global layers, q pre-scaled."""
    return AttnConfig(n_layers=n_layers, n_heads=8, n_kv_heads=4, head_dim=256, seq_len=seq_len,
                      rope_theta=1e6, rope_theta_swa=1e4, swa_theta_on_window_layers=1,
                      rope_style=ROPE_NEOX, scale_mode=SCALE_Q_PRESCALED, image_mode=IMAGE_BIDIRECTIONAL,
                      layer_windows=gemma_layer_windows(n_layers, window, 6), kv_format=kv_format, **kw)


def qwen25_14b_decode(n_layers=48, seq_len=131072, max_batch=16, kv_format=KV_BF16, **kw) -> AttnConfig:
    """Config 5: 40 query / 8 KV heads (GQA 5:1), head_dim 128, NeoX RoPE theta 1e6."""
    return AttnConfig(n_layers=n_layers, n_heads=40, n_kv_heads=8, head_dim=128, seq_len=seq_len,
                      max_batch=max_batch, rope_theta=1e6, rope_style=ROPE_NEOX, kv_format=kv_format, **kw)
