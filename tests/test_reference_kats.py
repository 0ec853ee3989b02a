"""Known-answer tests of the reference, restated against the CPU oracle and
against the host-side planners of the product library (no GPU needed).

Each test names the reference test it restates (paths inside
apimeister/gguf-runner). The constants are the reference's literals.
"""
import math

import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import (AttnConfig, KV_Q8_ROW, ROPE_ADJACENT, ROPE_INTERLEAVED, ROPE_NEOX)
from tests.oracle_binding import Oracle, OraclePlan, bf16_round, lib as oracle_lib


def fixture_config(**kw):
    """qwen3next_dense_test_fixture (src/engine/runtime/inference.rs:4328-4386): dim 4, one head, theta 1e4."""
    base = dict(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=4, seq_len=8, rope_dim=4, rope_theta=10000.0,
                rope_theta_swa=0.0, swa_pattern=0, rope_style=ROPE_ADJACENT, kv_format=KV_Q8_ROW)
    base.update(kw)
    return AttnConfig(**base)


# src/engine/runtime/inference.rs:4099-4118
def test_rope_scaling_switches_local_and_global_layers_at_the_same_position():
    cfg = fixture_config(n_layers=2, layer_windows=[1024, 0], rope_scale_global=0.125)
    ora = Oracle(cfg)
    for layer, angle in [(0, 8.0), (1, 1.0), (0, 8.0)]:
        q = np.zeros(4, np.float32)
        k = np.zeros(4, np.float32)
        q[0] = 1.0
        k[0] = 1.0
        ora.apply_rope_qk(layer, 8, q, k)
        for values in (q, k):
            assert abs(values[0] - np.float32(math.cos(angle))) < 1e-7
            assert abs(values[1] - np.float32(math.sin(angle))) < 1e-7


# src/engine/runtime/inference.rs:4121-4131
@pytest.mark.parametrize("scale", [0.0, -1.0, float("nan"), float("inf")])
def test_rope_scaling_rejects_invalid_runtime_policies(scale):
    with pytest.raises(ValueError):
        Oracle(fixture_config(rope_scale_global=scale, rope_scale_local=1.0))
    with pytest.raises(ValueError):
        Oracle(fixture_config(rope_scale_global=1.0, rope_scale_local=scale))


# src/engine/runtime/inference.rs:4134-4182
@pytest.mark.parametrize("head_dim,rope_dim,sections", [(128, 128, [24, 20, 20, 0]), (256, 64, [11, 11, 10, 0])])
def test_image_rope_rotates_reference_axes_and_preserves_partial_rope_tail(head_dim, rope_dim, sections):
    # rope_theta 1 makes every frequency 1, as the reference test does by filling the table
    cfg = fixture_config(head_dim=head_dim, rope_dim=rope_dim, rope_sections=sections, rope_layout=ROPE_INTERLEAVED,
                         rope_style=ROPE_NEOX, rope_theta=1.0)
    ora = Oracle(cfg)
    plan = OraclePlan()
    plan.append_text(2)
    plan.append_grid([1, 2, 3], 6)
    ora.set_position_plan(plan.positions, plan.next_text_position)
    half = rope_dim // 2
    q = np.zeros(head_dim, np.float32)
    q[:half] = 1.0
    q[rope_dim:] = 0.75
    k = q.copy()
    ora.apply_rope_qk(0, 7, q, k)
    # physical token 7 has logical T/H/W = (2, 3, 4)
    for i, cos, sin in [(0, -0.41614684, 0.9092974), (1, -0.9899925, 0.14112), (2, -0.6536436, -0.7568025)]:
        assert abs(q[i] - np.float32(cos)) < 1e-7
        assert abs(q[i + half] - np.float32(sin)) < 1e-7
    assert np.array_equal(q, k)
    assert np.all(q[rope_dim:] == 0.75)
    # the first decoded text token follows max(grid)+1, not KV row 8
    c, s = ora.rope_angles(0, 8)
    assert np.all(np.abs(c - np.float32(0.2836622)) < 1e-7)
    assert np.all(np.abs(s + np.float32(0.9589243)) < 1e-7)


def _plans():
    return [("oracle", OraclePlan), ("product", g.RopePositionPlan)]


# src/engine/positions.rs:79-107
@pytest.mark.parametrize("name,Plan", _plans())
def test_rectangular_grid_and_following_text_match_reference_positions(name, Plan):
    plan = Plan()
    plan.append_text(2)
    plan.append_grid([1, 2, 3], 6)
    plan.append_text(2)
    assert plan.positions == [[0, 0, 0], [1, 1, 1], [2, 2, 2], [2, 2, 3], [2, 2, 4], [2, 3, 2], [2, 3, 3],
                              [2, 3, 4], [5, 5, 5], [6, 6, 6]]
    assert plan.at(10) == [7, 7, 7]
    assert plan.at(12) == [9, 9, 9]
    plan.append_text(3)
    assert plan.at(12) == [9, 9, 9]
    assert plan.at(13) == [10, 10, 10]


# src/engine/positions.rs:110-121
@pytest.mark.parametrize("impl", ["oracle", "product"])
def test_interleaved_axes_match_reference_section_slices(impl):
    import ctypes as C

    def axis(layout, i, sections):
        if impl == "product":
            return g.rope_axis(layout, i, sections)
        sec = (C.c_int32 * 4)(*sections)
        return oracle_lib().ora_rope_axis(layout, i, sec)

    axes = [axis(1, i, [24, 20, 20, 0]) for i in range(64)]
    assert axes[:9] == [0, 1, 2, 0, 1, 2, 0, 1, 2]
    assert axes[57:] == [0, 1, 2, 0, 0, 0, 0]
    axes = [axis(1, i, [11, 11, 10, 0]) for i in range(32)]
    assert axes[27:] == [0, 1, 2, 0, 1]
    assert all(axis(0, i, [0, 0, 0, 0]) == 0 for i in range(64))


# src/engine/positions.rs:124-136
def test_invalid_grids_fail_before_modifying_positions():
    big = 2 ** 63 - 1
    for grid, count in [([0, 2, 3], 0), ([1, 2, 3], 5), ([big, 2, 2], 1)]:
        for Plan in (OraclePlan, g.RopePositionPlan):
            plan = Plan()
            failed = False
            try:
                failed = plan.append_grid(grid, count) not in (None, 0)
            except ValueError:
                failed = True
            assert failed
            assert len(plan) == 0 and plan.next_text_position == 0


# src/engine/runtime/attention.rs:104-174
@pytest.mark.parametrize("impl", ["oracle", "product"])
def test_image_attention_chunks_never_split_blocks(impl):
    import ctypes as C
    blocks = [(2, 5), (8, 4)]
    arr = np.array(blocks, dtype=np.int64)

    if impl == "product":
        plan = g.MediaAttentionPlan(12, blocks)
        block_at = plan.block_at

        def chunk_end(start, limit, chunk):
            return plan.chunk_end(start, limit, chunk)

        def invalid(bl):
            with pytest.raises(ValueError):
                g.MediaAttentionPlan(12, bl)
    else:
        L = oracle_lib()
        assert L.ora_media_plan_validate(C.c_void_p(arr.ctypes.data), 2, 12) == 0

        def block_at(pos):
            for s, n in blocks:
                if s <= pos < s + n:
                    return (s, n)
            return None

        def chunk_end(start, limit, chunk):
            r = L.ora_media_chunk_end(C.c_void_p(arr.ctypes.data), 2, 12, start, limit, min(chunk, 2 ** 63 - 1))
            if r < 0:
                raise ValueError("invalid")
            return r

        def invalid(bl):
            a = np.array(bl, dtype=np.uint64).astype(np.int64)
            assert L.ora_media_plan_validate(C.c_void_p(a.ctypes.data), len(bl), 12) != 0

    for chunk in [1, 2, 3, 4, 8, 2 ** 64 - 1]:
        start = 0
        while start < 12:
            end = chunk_end(start, 12, chunk)
            assert end > start
            b = block_at(start)
            if b is not None:
                assert (start, end) == (b[0], b[0] + b[1])
            else:
                assert all(block_at(p) is None for p in range(start, end))
            start = end
    for args in [(3, 12, 2), (2, 6, 2), (0, 12, 0), (0, 13, 1)]:
        with pytest.raises(ValueError):
            chunk_end(*args)
    for bl in [[(1, 0)], [(11, 2)], [(2 ** 63 - 1, 1)], [(2, 5), (6, 2)]]:
        invalid(bl)
    # default causal policy: visible_keys(plan, 0, 3) == 0..4
    ora = Oracle(fixture_config(seq_len=16))
    ora.set_media_blocks(blocks, 12)
    assert ora.visible_keys(0, 3) == range(0, 4)


# src/vendors/gemma.rs:383-420 (scalar period form): period 6 -> five local layers then one global
def test_gemma_window_pattern_period():
    import ctypes as C
    want = [1024 if l % 6 != 5 else 0 for l in range(12)]
    assert g.gemma_layer_windows(12, 1024, 6) == want
    out = np.zeros(12, np.int32)
    oracle_lib().ora_gemma_layer_windows(12, 1024, 6, C.c_void_p(out.ctypes.data))
    assert out.tolist() == want
    assert g.gemma_layer_windows(4, 512, 0) == [512] * 4   # period zero: every layer local
    assert g.gemma_layer_windows(4, 0, 6) == [0] * 4       # no window: every layer global


# window semantics of LanguageAttentionPolicy (src/engine/types.rs:612-620): the window counts the
# current token, a key at distance == window is excluded; bidirectional blocks override it
def test_visible_keys_window_and_block_override():
    cfg = fixture_config(n_layers=2, seq_len=32, layer_windows=[3, 0], image_mode=1)
    ora = Oracle(cfg)
    ora.set_media_blocks([(4, 6)], 16)
    assert ora.visible_keys(0, 2) == range(0, 3)
    assert ora.visible_keys(0, 3) == range(1, 4)
    assert ora.visible_keys(1, 3) == range(0, 4)
    # inside the block: every row of the block, plus the window reaching before it
    assert ora.visible_keys(0, 4) == range(2, 10)
    assert ora.visible_keys(0, 9) == range(4, 10)
    assert ora.visible_keys(1, 7) == range(0, 10)
    assert ora.visible_keys(0, 10) == range(8, 11)


# src/engine/runtime/inference.rs:251-267: zero row -> scale 1 and zero codes; half rounds away from zero
def test_q8_row_quantiser_edges():
    cfg = fixture_config(head_dim=8, rope_dim=8, n_kv_heads=1, seq_len=4)
    ora = Oracle(cfg)
    ora.kv_write_token(0, 0, np.zeros(8, np.float32), np.zeros(8, np.float32))
    kq, vq, ks, vs = ora.kv_read_q8(0, 0)
    assert ks[0] == 1.0 and vs[0] == 1.0 and not kq.any() and not vq.any()
    k = np.array([127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -127.0, 0.0], np.float32)
    ora.kv_write_token(0, 1, k, k)
    kq, _, ks, _ = ora.kv_read_q8(0, 1)
    assert ks[0] == 1.0
    assert kq.tolist() == [127, 1, -1, 2, -2, 3, -127, 0]


# online and two-pass softmax are the same function up to rounding
# (src/engine/runtime/inference.rs:2320-2429 vs :2430-2527)
@pytest.mark.parametrize("kv_format", [0, 1, 2, 3])
def test_oracle_online_matches_two_pass_and_naive(kv_format):
    rng = np.random.default_rng(7)
    base = dict(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=32, seq_len=40, rope_dim=0, rope_theta=1e6,
                rope_style=ROPE_NEOX, kv_format=kv_format)
    a = Oracle(AttnConfig(softmax_mode=0, **base))
    b = Oracle(AttnConfig(softmax_mode=1, **base))
    m = 40
    q = rng.standard_normal((m, 128)).astype(np.float32)
    k = rng.standard_normal((m, 64)).astype(np.float32)
    v = rng.standard_normal((m, 64)).astype(np.float32)
    oa = a.prefill(0, 0, q, k, v)
    ob = b.prefill(0, 0, q, k, v)
    assert np.max(np.abs(oa - ob)) < 2e-6
    # naive float64 softmax over the oracle's own stored rows
    last = m - 1
    qr = q[last].copy()
    kr = k[last].copy()
    a.apply_rope_qk(0, last, qr, kr)
    rows = [a.kv_read_row(0, t) for t in range(m)]
    K = np.stack([r[0] for r in rows]).astype(np.float64).reshape(m, 2, 32)
    V = np.stack([r[1] for r in rows]).astype(np.float64).reshape(m, 2, 32)
    out = np.zeros(128)
    for h in range(4):
        s = K[:, h // 2, :] @ qr[h * 32:(h + 1) * 32].astype(np.float64) / math.sqrt(32)
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h * 32:(h + 1) * 32] = p @ V[:, h // 2, :]
    assert np.max(np.abs(out - oa[last])) < 1e-5


def test_bf16_rounding_helpers_agree():
    rng = np.random.default_rng(3)
    x = rng.standard_normal(1000).astype(np.float32)
    L = oracle_lib()
    want = np.array([L.ora_bf16_to_f32(L.ora_f32_to_bf16(float(v))) for v in x], np.float32)
    assert np.array_equal(bf16_round(x), want)


# ---- TurboQuant cache format (src/engine/runtime/inference.rs:349-1334) ----

def _splitmix64(x):
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def _turbo_oracle(head_dim, n_layers=3, n_kv_heads=8, **kw):
    cfg = AttnConfig(n_layers=n_layers, n_heads=n_kv_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=8,
                     rope_dim=head_dim, rope_theta=1e6, rope_style=ROPE_NEOX, kv_format=4, **kw)
    return Oracle(cfg), cfg


# inference.rs:4546-4556: forward then inverse rotation restores the vector (power-of-two head: FWHT included)
def test_turboquant_transform_is_self_inverse_for_power_of_two_heads():
    ora, _ = _turbo_oracle(8)
    values = np.array([0.25, -0.5, 1.0, -1.5, 0.75, 0.125, -0.25, 0.5], np.float32)
    fwd = ora.turbo_transform(2, 3, 0, 1, values)
    assert np.max(np.abs(fwd - values)) > 1e-3
    back = ora.turbo_transform(2, 3, 1, 0, fwd)
    assert np.max(np.abs(back - values)) < 1e-5


# inference.rs:4558-4566: a head that is not a power of two skips the FWHT (only the sign flips remain)
def test_turboquant_transform_is_self_inverse_for_non_power_of_two_heads():
    ora, _ = _turbo_oracle(6, n_layers=2, n_kv_heads=8)
    values = np.array([0.25, -0.5, 1.0, -1.5, 0.75, 0.125], np.float32)
    fwd = ora.turbo_transform(1, 7, 2, 3, values)
    assert np.array_equal(np.abs(fwd), np.abs(values))
    back = ora.turbo_transform(1, 7, 3, 2, fwd)
    assert np.max(np.abs(back - values)) < 1e-6


# inference.rs:370-395 and :4292-4304: element i is negated iff splitmix64(seed ^ i) & 1, seed from (layer, head, salt)
def test_turboquant_sign_pattern_follows_splitmix64():
    ora, _ = _turbo_oracle(6, n_layers=2, n_kv_heads=8)
    salts = [0x9E3779B97F4A7C15, 0xC2B2AE3D27D4EB4F, 0x165667B19E3779F9, 0xD6E8FEB86659FD93]
    ones = np.ones(6, np.float32)
    for layer, head in ((0, 0), (1, 7)):
        for a, b in ((0, 1), (2, 3)):
            got = ora.turbo_transform(layer, head, a, b, ones)  # no FWHT at length 6: product of both sign vectors
            want = np.ones(6, np.float32)
            for slot in (a, b):
                seed = _splitmix64(((layer << 32) ^ head ^ salts[slot]) & ((1 << 64) - 1))
                want *= np.array([-1.0 if _splitmix64(seed ^ i) & 1 else 1.0 for i in range(6)], np.float32)
            assert np.array_equal(got, want)


# inference.rs:885-952: codes follow the +-0.9815985 / 0 thresholds of r / sigma, zero rows store zero codes, all
# sign bits set and zero norms; codes are packed four per byte, LSB first (:853-855, :4535-4545)
def test_turboquant_write_codes_and_zero_row():
    ora, cfg = _turbo_oracle(16, n_layers=1, n_kv_heads=2)
    rng = np.random.default_rng(3)
    k = rng.standard_normal(32).astype(np.float32)
    v = np.zeros(32, np.float32)
    ora.kv_write_token(0, 0, k, v)
    row = ora.kv_read_turbo(0, 0)
    assert not row["v_base"].any() and (row["v_sign"] == 0xFF).all()
    assert (row["v_scale"] == 0).all() and (row["v_rnorm"] == 0).all()
    centroids = np.array([-1.510417, -0.45278, 0.45278, 1.510417], np.float32)
    for h in range(2):
        r = ora.turbo_transform(0, h, 0, 1, k[h * 16:(h + 1) * 16])
        sigma = np.float32(np.sqrt(np.sum(r.astype(np.float32) ** 2, dtype=np.float32)) / np.float32(4.0))
        assert abs(row["k_scale"][h] - sigma) <= 1e-6 * sigma
        codes = [(row["k_base"][(h * 16 + i) // 4] >> (((h * 16 + i) & 3) * 2)) & 3 for i in range(16)]
        x = r / row["k_scale"][h]
        want = [0 if t < -0.9815985 else 1 if t < 0 else 2 if t < 0.9815985 else 3 for t in x]
        assert codes == want
        resid = r - centroids[codes] * row["k_scale"][h]
        gamma = np.sqrt(np.sum(resid.astype(np.float64) ** 2))
        assert abs(row["k_rnorm"][h] - gamma) < 1e-5
        proj = ora.turbo_transform(0, h, 2, 3, (resid / row["k_rnorm"][h]).astype(np.float32))
        bits = [(row["k_sign"][(h * 16 + i) // 8] >> ((h * 16 + i) & 7)) & 1 for i in range(16)]
        assert bits == [1 if p >= 0 else 0 for p in proj]


# the format is lossy by design: its attention output stays close to the f32 cache's, and the online and two-pass
# arms (:2320-2429, :2430-2527) agree with each other
def test_turboquant_attention_tracks_f32_attention():
    rng = np.random.default_rng(11)
    base = dict(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=64, seq_len=48, rope_dim=0, rope_theta=1e6,
                rope_style=ROPE_NEOX)
    m = 48
    q = rng.standard_normal((m, 256)).astype(np.float32)
    k = rng.standard_normal((m, 128)).astype(np.float32)
    v = rng.standard_normal((m, 128)).astype(np.float32)
    exact = Oracle(AttnConfig(kv_format=0, **base)).prefill(0, 0, q, k, v)
    two_pass = Oracle(AttnConfig(kv_format=4, softmax_mode=0, **base)).prefill(0, 0, q, k, v)
    online = Oracle(AttnConfig(kv_format=4, softmax_mode=1, **base)).prefill(0, 0, q, k, v)
    assert np.max(np.abs(two_pass - online)) < 5e-6
    err = np.abs(two_pass - exact)
    assert err.max() < 1.5 and np.sqrt(np.mean(err ** 2)) < 0.35
