"""Output gate (Qwen3Next / Qwen3.5) and row-range export / import of the quantised caches.

Gate: src/engine/runtime/inference.rs:3509-3519 (sigmoid_mul_inplace per head on the second halves of the
packed q / gate projection, then sanitize_finite_inplace). Cache I/O: the sections of the reference's prefill
cache blob, src/app/prefill_cache.rs:11-19.
"""
import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import AttnConfig, GgrError, KV_BF16, KV_F32, KV_Q8_BLOCK32, KV_Q8_ROW, KV_TURBO
from tests.oracle_binding import Oracle, bf16_bits, bf16_round

pytestmark = pytest.mark.gpu
THREADS = 8
TOL = {KV_F32: 1e-3, KV_Q8_ROW: 1e-3, KV_BF16: 2e-2, KV_TURBO: 2e-2}


def rand(rng, *shape):
    return rng.standard_normal(shape).astype(np.float32)


@pytest.mark.parametrize("kv_format,n_heads,n_kv_heads,head_dim", [(KV_F32, 4, 2, 64), (KV_Q8_ROW, 16, 8, 128),
                                                                  (KV_BF16, 32, 4, 128), (KV_BF16, 8, 4, 256),
                                                                  (KV_TURBO, 8, 2, 128)])
@pytest.mark.parametrize("packed", [False, True])
def test_output_gate_matches_oracle(kv_format, n_heads, n_kv_heads, head_dim, packed):
    B, m = 2, 300
    cfg = AttnConfig(n_layers=1, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=512, max_batch=B,
                     rope_theta=1e6, kv_format=kv_format)
    ctx, ora = g.AttnContext(cfg), Oracle(cfg, threads=THREADS)
    rng = np.random.default_rng(head_dim + n_heads)
    stride = 2 * head_dim if packed else head_dim
    tol = TOL[kv_format]

    def gate_rows(n):
        # the packed layout carries q in the first half of each head's 2 * head_dim span and the gate in the second
        buf = rand(rng, n, n_heads * stride) * 3.0
        view = buf.reshape(-1)[head_dim:] if packed else buf.reshape(-1)
        view[1] = np.inf   # gate -> sigmoid 1
        view[2] = -np.inf  # gate -> sigmoid 0
        view[3] = np.nan   # product is not finite -> 0
        return buf, view

    # prefill rows (f32 inputs)
    q, k, v = rand(rng, m, cfg.q_dim), rand(rng, m, cfg.kv_dim), rand(rng, m, cfg.kv_dim)
    _buf, gate = gate_rows(m)
    want = ora.sigmoid_gate(ora.prefill(0, 0, q, k, v), gate, stride)
    got = ctx.prefill_gated(0, 0, q, k, v, gate, stride)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - want)) <= tol
    # decode steps, both sequences
    ora.prefill(0, 0, q[:50], k[:50], v[:50], seq=1)
    ctx.prefill(0, 0, q[:50], k[:50], v[:50], seq=1)
    for step in range(2):
        pos = [m + step, 50 + step]
        q1, k1, v1 = rand(rng, B, cfg.q_dim), rand(rng, B, cfg.kv_dim), rand(rng, B, cfg.kv_dim)
        _buf, gate = gate_rows(B)
        want = ora.sigmoid_gate(ora.decode(0, pos, q1, k1, v1), gate, stride)
        got = ctx.decode_gated(0, pos, q1, k1, v1, gate, stride)
        assert np.max(np.abs(got - want)) <= tol
        assert got[0, 3] == 0.0 and got[0, 2] == 0.0
    ctx.close()


def test_output_gate_bf16_rows_on_device_pointers():
    import torch
    m = 384
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=512, rope_theta=1e6, kv_format=KV_BF16)
    ctx, ora = g.AttnContext(cfg), Oracle(cfg, threads=THREADS)
    rng = np.random.default_rng(12)
    q, k, v, gate = (bf16_round(rand(rng, m, d)) for d in (cfg.q_dim, cfg.kv_dim, cfg.kv_dim, cfg.q_dim))
    want = ora.sigmoid_gate(ora.prefill(0, 0, q, k, v), gate)
    tq, tk, tv, tg = (torch.from_numpy(x).cuda().to(torch.bfloat16) for x in (q, k, v, gate))
    got = ctx.prefill_gated(0, 0, tq, tk, tv, tg).cpu().numpy()
    assert np.max(np.abs(got - want)) <= 2e-2
    # host bf16 bit patterns through the pipelined host-buffer path
    got_h = ctx.prefill_gated(0, 0, bf16_bits(q), bf16_bits(k), bf16_bits(v), bf16_bits(gate))
    assert np.max(np.abs(got_h - want)) <= 2e-2
    with pytest.raises(GgrError):
        ctx.prefill_gated(0, 0, tq, tk, tv, tg, gate_head_stride=64)
    ctx.close()


def test_q8_block_scales_export_import_round_trip():
    cfg = AttnConfig(n_layers=2, n_heads=8, n_kv_heads=4, head_dim=64, seq_len=64, rope_theta=1e6,
                     kv_format=KV_Q8_BLOCK32)
    rng = np.random.default_rng(6)
    q, k, v = rand(rng, 40, cfg.q_dim), rand(rng, 40, cfg.kv_dim), rand(rng, 40, cfg.kv_dim)
    ora = Oracle(cfg, threads=2)
    ora.prefill(1, 0, q, k, v)
    with g.AttnContext(cfg) as a, g.AttnContext(cfg) as b:
        a.prefill(1, 0, q, k, v)
        kq, vq, ks, vs = a.kv_export(1, 5, 30)
        assert ks.shape == (30, cfg.kv_dim // 32)
        for row in (5, 20, 34):
            okq, ovq, oks, ovs = ora.kv_read_q8(1, row)
            assert np.array_equal(kq[row - 5], okq) and np.array_equal(vq[row - 5], ovq)
            assert np.array_equal(ks[row - 5], oks) and np.array_equal(vs[row - 5], ovs)
        b.kv_import(1, 5, kq, vq, ks, vs)
        for row in (5, 34):
            ka, va = a.kv_read_row(1, row)
            kb, vb = b.kv_read_row(1, row)
            assert np.array_equal(ka, kb) and np.array_equal(va, vb)


def test_turboquant_sections_export_import_round_trip():
    cfg = AttnConfig(n_layers=2, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=256, rope_theta=1e6, kv_format=KV_TURBO)
    rng = np.random.default_rng(8)
    n = 200
    q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
    ora = Oracle(cfg, threads=THREADS)
    ora.prefill(1, 0, q, k, v)
    with g.AttnContext(cfg) as a, g.AttnContext(cfg) as b:
        a.prefill(1, 0, q, k, v)
        sec = a.kv_export_turbo(1, 10, 150)
        assert sec["k_base"].shape == (150, cfg.kv_dim // 4) and sec["k_sign"].shape == (150, cfg.kv_dim // 8)
        assert sec["k_scale"].shape == (150, cfg.n_kv_heads)
        for row in (10, 99, 159):
            one = a.kv_read_turbo(1, row)
            want = ora.kv_read_turbo(1, row)
            for name, arr in sec.items():
                assert np.array_equal(arr[row - 10], one[name]), name
            # value rows see bit-identical inputs on both sides
            for name in ("v_base", "v_sign", "v_scale", "v_rnorm"):
                assert np.array_equal(sec[name][row - 10], want[name]), name
        b.kv_import_turbo(1, 10, sec)
        # rows 10..159 now live in b: attention restricted to them agrees bit for bit
        b.kv_import_turbo(1, 0, a.kv_export_turbo(1, 0, 10))
        q1, k1, v1 = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
        assert np.array_equal(a.decode(1, [160], q1, k1, v1), b.decode(1, [160], q1, k1, v1))
        with pytest.raises(GgrError):
            a.kv_export(1, 0, 4)
    with g.AttnContext(AttnConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=64, seq_len=8, kv_format=KV_F32)) as c:
        with pytest.raises(GgrError):
            c.kv_export_turbo(0, 0, 1)
