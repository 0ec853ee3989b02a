"""The matmuls either side of the attention path on the device, against the reference's scalar matmul.

ggr_proj_matmul replaces matmul_quantized_with_scratch (src/engine/kernels/quant.rs:7225) for F32, BF16, Q8_0,
Q4_K and Q6_K weights; ggr_attn_layer_decode / ggr_attn_layer_prefill run q / k / v projections, the attention path and the output
projection (src/engine/runtime/inference.rs:3144-3527) with only hidden-state rows crossing the boundary. Up to 16
rows use f32 arithmetic (relative tolerance 1e-3 of the output scale), more rows the tensor cores with bf16 operands
(2e-2).
"""
import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import (AttnConfig, GgrError, KV_BF16, KV_F32, KV_Q8_ROW, W_BF16, W_F32, W_Q4_K, W_Q6_K,
                                      W_Q8_0, Weights)
from tests.oracle_binding import Oracle, bf16_bits, matmul as ora_matmul, quantize_q4_k, quantize_q6_k, quantize_q8_0

pytestmark = pytest.mark.gpu


def make_weights(rng, wtype, rows, cols):
    """(device weights, raw bytes for the oracle) of a random matrix scaled like a projection (1 / sqrt(cols))."""
    w = (rng.standard_normal((rows, cols)) / np.sqrt(cols)).astype(np.float32)
    raw = {W_F32: lambda: w, W_BF16: lambda: bf16_bits(w), W_Q8_0: lambda: quantize_q8_0(w), W_Q4_K: lambda: quantize_q4_k(w),
           W_Q6_K: lambda: quantize_q6_k(w)}[wtype]()
    return Weights(wtype, rows, cols, raw), np.ascontiguousarray(raw)


@pytest.mark.parametrize("wtype", [W_F32, W_BF16, W_Q8_0, W_Q4_K, W_Q6_K])
@pytest.mark.parametrize("rows,cols,n", [(64, 256, 1), (1024, 1024, 3), (2048, 4096, 16), (1000, 1056, 7)])
def test_weight_streaming_matmul_matches_reference(wtype, rows, cols, n):
    if wtype in (W_Q4_K, W_Q6_K) and cols % 256:
        cols = 1280   # K-quant rows are whole super-blocks of 256
    rng = np.random.default_rng(rows + cols + n)
    cfg = AttnConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=64, seq_len=16, kv_format=KV_F32)
    w, raw = make_weights(rng, wtype, rows, cols)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    want = ora_matmul(wtype, rows, cols, raw, x)
    with g.AttnContext(cfg) as ctx:
        got = ctx.proj_matmul(w, x)
    assert np.max(np.abs(got - want)) <= 1e-3 * max(1.0, float(np.max(np.abs(want))))
    w.close()


@pytest.mark.parametrize("wtype", [W_BF16, W_Q8_0, W_F32, W_Q4_K, W_Q6_K])
@pytest.mark.parametrize("rows,cols,n", [(256, 256, 128), (4096, 1024, 300), (1000, 1056, 130), (512, 4096, 17)])
def test_tensor_core_matmul_matches_reference(wtype, rows, cols, n):
    import torch
    if wtype in (W_Q4_K, W_Q6_K) and cols % 256:
        cols = 1280
    rng = np.random.default_rng(rows + cols + n)
    cfg = AttnConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=64, seq_len=16, kv_format=KV_F32)
    w, raw = make_weights(rng, wtype, rows, cols)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    want = ora_matmul(wtype, rows, cols, raw, x[::7])   # every 7th row through the scalar reference
    with g.AttnContext(cfg) as ctx:
        got = ctx.proj_matmul(w, x)
        got_dev = ctx.proj_matmul(w, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, got_dev)
    assert np.max(np.abs(got[::7] - want)) <= 2e-2 * max(1.0, float(np.max(np.abs(want))))
    assert np.all(np.isfinite(got))
    w.close()


def reference_layer(ora, layer, pos_list, xb, raws, wtypes, dims, prefill_base=None):
    """The reference composition: projections, attention, output projection, non-finite values zeroed."""
    (q_dim, kv_dim, dim) = dims
    q = ora_matmul(wtypes[0], q_dim, dim, raws[0], xb)
    k = ora_matmul(wtypes[1], kv_dim, dim, raws[1], xb)
    v = ora_matmul(wtypes[2], kv_dim, dim, raws[2], xb)
    att = ora.prefill(layer, prefill_base, q, k, v) if prefill_base is not None else ora.decode(layer, pos_list, q, k, v)
    out = ora_matmul(wtypes[3], dim, q_dim, raws[3], att)
    out[~np.isfinite(out)] = 0.0
    return out


@pytest.mark.parametrize("wtype,kv_format,tol", [(W_Q8_0, KV_Q8_ROW, 2e-3), (W_BF16, KV_F32, 2e-3), (W_Q8_0, KV_BF16, 2e-2),
                                                  (W_Q4_K, KV_F32, 2e-3), (W_Q6_K, KV_Q8_ROW, 2e-3)])
def test_layer_decode_and_prefill_match_reference(wtype, kv_format, tol):
    # Qwen3-0.6B-shaped attention half-layer: hidden 1024, 16 query / 8 kv heads of 128
    dim, B = 1024, 2
    cfg = AttnConfig(n_layers=2, n_heads=16, n_kv_heads=8, head_dim=128, seq_len=256, max_batch=B, rope_theta=1e6,
                     kv_format=kv_format)
    rng = np.random.default_rng(31 + wtype + kv_format)
    shapes = [(cfg.q_dim, dim), (cfg.kv_dim, dim), (cfg.kv_dim, dim), (dim, cfg.q_dim)]
    ws, raws = zip(*[make_weights(rng, wtype, r, c) for r, c in shapes])
    wtypes, dims = [wtype] * 4, (cfg.q_dim, cfg.kv_dim, dim)
    ctx, ora = g.AttnContext(cfg), Oracle(cfg, threads=8)
    # a prompt chunk per sequence: 12 rows take the weight-streaming kernel, 150 rows the tensor cores (bf16 operands)
    for seq, m in ((0, 12), (1, 150)):
        xb = rng.standard_normal((m, dim)).astype(np.float32)
        q = ora_matmul(wtype, cfg.q_dim, dim, raws[0], xb)
        k = ora_matmul(wtype, cfg.kv_dim, dim, raws[1], xb)
        v = ora_matmul(wtype, cfg.kv_dim, dim, raws[2], xb)
        att = ora.prefill(1, 0, q, k, v, seq=seq)
        want = ora_matmul(wtype, dim, cfg.q_dim, raws[3], att)
        got = ctx.layer_prefill(1, 0, xb, *ws, seq=seq)
        scale = max(1.0, float(np.max(np.abs(want))))
        assert np.max(np.abs(got - want)) <= (tol if m <= 16 else 2e-2) * scale, (seq, m)
    for step in range(2):
        pos = [12 + step, 150 + step]
        xb = rng.standard_normal((B, dim)).astype(np.float32)
        want = reference_layer(ora, 1, pos, xb, raws, wtypes, dims)
        got = ctx.layer_decode(1, pos, xb, *ws)
        # sequence 1 attends over rows that went through bf16 projections on the device
        assert np.max(np.abs(got[0] - want[0])) <= tol * max(1.0, float(np.max(np.abs(want))))
        assert np.max(np.abs(got[1] - want[1])) <= 2e-2 * max(1.0, float(np.max(np.abs(want))))
    with pytest.raises(GgrError):
        ctx.layer_decode(1, [0, 0], xb, ws[1], ws[1], ws[2], ws[3])   # wq with the wrong row count
    ctx.close()
    for w in ws:
        w.close()


def test_layer_decode_with_mixed_weight_types():
    """A Q4_K_M-style layer: wq / wk in Q4_K, wv in Q6_K, wo in Q8_0. The three input projections then run as
    separate launches (one launch serves several matrices only when their types agree); the result is the
    reference composition of the four matmuls around the path."""
    dim, B = 1024, 3
    cfg = AttnConfig(n_layers=1, n_heads=16, n_kv_heads=8, head_dim=128, seq_len=64, max_batch=B, rope_theta=1e6,
                     kv_format=KV_F32)
    rng = np.random.default_rng(91)
    wtypes = [W_Q4_K, W_Q4_K, W_Q6_K, W_Q8_0]
    shapes = [(cfg.q_dim, dim), (cfg.kv_dim, dim), (cfg.kv_dim, dim), (dim, cfg.q_dim)]
    ws, raws = zip(*[make_weights(rng, t, r, c) for t, (r, c) in zip(wtypes, shapes)])
    ctx, ora = g.AttnContext(cfg), Oracle(cfg, threads=8)
    for step in range(3):
        pos = [step] * B
        xb = rng.standard_normal((B, dim)).astype(np.float32)
        want = reference_layer(ora, 0, pos, xb, raws, wtypes, (cfg.q_dim, cfg.kv_dim, dim))
        got = ctx.layer_decode(0, pos, xb, *ws)
        assert np.max(np.abs(got - want)) <= 2e-3 * max(1.0, float(np.max(np.abs(want))))
    ctx.close()
    for w in ws:
        w.close()


def test_weight_upload_rejects_bad_shapes():
    with pytest.raises(GgrError):
        Weights(W_Q8_0, 64, 48, np.zeros(64 * 34, np.uint8))        # Q8_0 needs cols % 32 == 0
    with pytest.raises(GgrError):
        Weights(W_Q4_K, 64, 384, np.zeros(64 * 144, np.uint8))      # K-quant rows are whole super-blocks of 256
    with pytest.raises(GgrError):
        Weights(W_Q6_K, 60, 256, np.zeros(60 * 210, np.uint8))      # rows must be a multiple of 8
    with pytest.raises(ValueError):
        Weights(W_BF16, 64, 64, np.zeros(10, np.uint16))
