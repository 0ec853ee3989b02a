"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same
seeded inputs. Tolerances: max abs error <= 1e-3 for f32 and q8 caches,
<= 2e-2 where operands are bf16."""
import math

import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200 import presets
from gguf_runner_b200.binding import (AttnConfig, GgrError, IMPL_AUTO, IMPL_MMA, IMPL_SIMT, KV_BF16, KV_F32, KV_Q8_BLOCK32,
                                      KV_Q8_ROW, KV_TURBO, ROPE_ADJACENT, ROPE_INTERLEAVED, ROPE_NEOX, SCALE_Q_PRESCALED,
                                      SHARD_KV_SEQUENCE)
from tests.oracle_binding import Oracle, bf16_bits, bf16_round

pytestmark = pytest.mark.gpu

TOL = {KV_F32: 1e-3, KV_Q8_ROW: 1e-3, KV_Q8_BLOCK32: 1e-3, KV_BF16: 2e-2, KV_TURBO: 1e-3}
THREADS = 8


def rand(rng, *shape):
    return rng.standard_normal(shape).astype(np.float32)


def make(cfg, plan=None, blocks=None, prompt_tokens=0):
    ctx = g.AttnContext(cfg)
    ora = Oracle(cfg, threads=THREADS)
    if plan is not None:
        ctx.set_position_plan(plan)
        ora.set_position_plan(plan.positions, plan.next_text_position)
    if blocks is not None:
        ctx.set_media_blocks(blocks, prompt_tokens)
        ora.set_media_blocks(blocks, prompt_tokens)
    return ctx, ora


def check_prefill_then_decode(cfg, m, steps, seed=0, layer=0, chunk=None, tol=None):
    rng = np.random.default_rng(seed)
    ctx, ora = make(cfg)
    tol = tol or TOL[cfg.kv_format]
    worst = 0.0
    pos = 0
    for c0 in range(0, m, chunk or m):
        n = min(chunk or m, m - c0)
        q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
        got = ctx.prefill(layer, pos, q, k, v)
        want = ora.prefill(layer, pos, q, k, v)
        worst = max(worst, float(np.max(np.abs(got - want))))
        pos += n
    for _ in range(steps):
        q, k, v = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
        got = ctx.decode(layer, [pos], q, k, v)
        want = ora.decode(layer, [pos], q, k, v)
        worst = max(worst, float(np.max(np.abs(got - want))))
        pos += 1
    assert worst <= tol, f"max abs err {worst} > {tol}"
    ctx.close()
    return worst


# ---- RoPE known answers on the device (restating src/engine/runtime/inference.rs:4099-4182) --------

def test_rope_scaling_local_and_global_layers_on_device():
    # head_dim 8 instead of the fixture's 4 (the device kernels need head_dim % 8 == 0); frequency 0 is still 1
    cfg = AttnConfig(n_layers=2, n_heads=1, n_kv_heads=1, head_dim=8, seq_len=16, rope_theta=10000.0,
                     rope_theta_swa=0.0, swa_pattern=0, rope_style=ROPE_ADJACENT, layer_windows=[1024, 0],
                     rope_scale_global=0.125)
    with g.AttnContext(cfg) as ctx:
        for layer, angle in [(0, 8.0), (1, 1.0), (0, 8.0)]:
            q = np.zeros(8, np.float32)
            k = np.zeros(8, np.float32)
            q[0] = k[0] = 1.0
            ctx.apply_rope_qk(layer, 8, q, k)
            for values in (q, k):
                assert abs(values[0] - math.cos(angle)) < 5e-7
                assert abs(values[1] - math.sin(angle)) < 5e-7


@pytest.mark.parametrize("head_dim,rope_dim,sections", [(128, 128, [24, 20, 20, 0]), (256, 64, [11, 11, 10, 0])])
def test_image_rope_axes_and_partial_tail_on_device(head_dim, rope_dim, sections):
    cfg = AttnConfig(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=head_dim, rope_dim=rope_dim, seq_len=16,
                     rope_theta=1.0, rope_sections=sections, rope_layout=ROPE_INTERLEAVED, rope_style=ROPE_NEOX,
                     swa_pattern=0)
    plan = g.RopePositionPlan()
    plan.append_text(2)
    plan.append_grid([1, 2, 3], 6)
    with g.AttnContext(cfg) as ctx:
        ctx.set_position_plan(plan)
        half = rope_dim // 2
        q = np.zeros(head_dim, np.float32)
        q[:half] = 1.0
        q[rope_dim:] = 0.75
        k = q.copy()
        ctx.apply_rope_qk(0, 7, q, k)
        for i, cos, sin in [(0, -0.41614684, 0.9092974), (1, -0.9899925, 0.14112), (2, -0.6536436, -0.7568025)]:
            assert abs(q[i] - cos) < 5e-7
            assert abs(q[i + half] - sin) < 5e-7
        assert np.array_equal(q, k)
        assert np.all(q[rope_dim:] == 0.75)
        # decode after the grid continues at max(grid) + 1: angle 5 on every frequency
        q2 = np.zeros(head_dim, np.float32)
        q2[:half] = 1.0
        k2 = q2.copy()
        ctx.apply_rope_qk(0, 8, q2, k2)
        assert np.all(np.abs(q2[:half] - 0.2836622) < 5e-7)
        assert np.all(np.abs(q2[half:rope_dim] + 0.9589243) < 5e-7)


@pytest.mark.parametrize("style", [ROPE_NEOX, ROPE_ADJACENT])
@pytest.mark.parametrize("pos", [0, 1, 777, 131071])
def test_rope_matches_oracle(style, pos):
    cfg = AttnConfig(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=64, seq_len=131072, rope_theta=1e6,
                     rope_style=style, kv_format=KV_BF16)
    rng = np.random.default_rng(pos)
    with g.AttnContext(cfg) as ctx:
        ora = Oracle(cfg)
        q, k = rand(rng, cfg.q_dim), rand(rng, cfg.kv_dim)
        q2, k2 = q.copy(), k.copy()
        ctx.apply_rope_qk(0, pos, q, k)
        ora.apply_rope_qk(0, pos, q2, k2)
        assert np.max(np.abs(q - q2)) < 2e-6
        assert np.max(np.abs(k - k2)) < 2e-6


# ---- append parity ---------------------------------------------------------------------------------

@pytest.mark.parametrize("kv_format", [KV_F32, KV_BF16, KV_Q8_ROW, KV_Q8_BLOCK32])
def test_kv_write_token_matches_oracle(kv_format):
    cfg = AttnConfig(n_layers=2, n_heads=8, n_kv_heads=4, head_dim=64, seq_len=8, kv_format=kv_format)
    rng = np.random.default_rng(11)
    with g.AttnContext(cfg) as ctx:
        ora = Oracle(cfg)
        for pos in range(4):
            k, v = rand(rng, cfg.kv_dim), rand(rng, cfg.kv_dim)
            if pos == 2:
                k[:] = 0.0  # all-zero row: scale 1, zero codes
            ctx.kv_write_token(1, pos, k, v)
            ora.kv_write_token(1, pos, k, v)
            gk, gv = ctx.kv_read_row(1, pos)
            wk, wv = ora.kv_read_row(1, pos)
            # same input, same rounding rule: the stored rows are identical
            assert np.array_equal(gk, wk) and np.array_equal(gv, wv)
        if kv_format == KV_Q8_ROW:
            kq, vq, ks, vs = ctx.kv_export(1, 0, 4)
            for pos in range(4):
                okq, ovq, oks, ovs = ora.kv_read_q8(1, pos)
                assert np.array_equal(kq[pos], okq) and np.array_equal(vq[pos], ovq)
                assert ks[pos] == oks[0] and vs[pos] == ovs[0]
            assert ks[2] == 1.0 and not kq[2].any()


def test_kv_export_import_round_trip():
    cfg = AttnConfig(n_layers=2, n_heads=4, n_kv_heads=2, head_dim=32, seq_len=16, kv_format=KV_Q8_ROW)
    rng = np.random.default_rng(5)
    with g.AttnContext(cfg) as a, g.AttnContext(cfg) as b:
        q, k, v = rand(rng, 10, cfg.q_dim), rand(rng, 10, cfg.kv_dim), rand(rng, 10, cfg.kv_dim)
        a.prefill(1, 0, q, k, v)
        rows = a.kv_export(1, 0, 10)
        b.kv_import(1, 0, *rows)
        q1, k1, v1 = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
        oa = a.decode(1, [10], q1, k1, v1)
        ob = b.decode(1, [10], q1, k1, v1)
        assert np.array_equal(oa, ob)


# ---- attention parity, small shapes ------------------------------------------------------------------

@pytest.mark.parametrize("kv_format", [KV_F32, KV_BF16, KV_Q8_ROW, KV_Q8_BLOCK32])
@pytest.mark.parametrize("head_dim,n_heads,n_kv_heads", [(32, 4, 4), (64, 8, 4), (128, 10, 2), (128, 16, 2),
                                                         (256, 8, 4), (96, 6, 2)])
def test_prefill_and_decode_match_oracle(kv_format, head_dim, n_heads, n_kv_heads):
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=160,
                     rope_theta=1e6, kv_format=kv_format)
    check_prefill_then_decode(cfg, m=131, steps=3, seed=head_dim + n_heads, layer=1, chunk=50)


@pytest.mark.parametrize("kv_format", [KV_F32, KV_Q8_ROW, KV_BF16])
def test_head_dim_8_matches_oracle(kv_format):
    # the shape of the reference's own chunked-prefill test (head_dim 8, rope_dim 6, one head)
    cfg = AttnConfig(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=8, rope_dim=6, seq_len=16, rope_theta=1e4,
                     rope_sections=[1, 1, 1, 0], rope_layout=ROPE_INTERLEAVED, kv_format=kv_format, swa_pattern=0)
    check_prefill_then_decode(cfg, m=10, steps=2, seed=1, chunk=4)


@pytest.mark.parametrize("window", [1, 3, 64])
@pytest.mark.parametrize("kv_format", [KV_F32, KV_BF16])
def test_sliding_window_matches_oracle(window, kv_format):
    cfg = AttnConfig(n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, seq_len=256, rope_theta=1e4,
                     layer_windows=[window, 0], kv_format=kv_format)
    check_prefill_then_decode(cfg, m=150, steps=3, seed=window, layer=0, chunk=64)
    check_prefill_then_decode(cfg, m=150, steps=3, seed=window, layer=1, chunk=64)


def test_gemma_mode_matches_oracle():
    # q pre-scaled, theta_swa on window layers, local / global rope scales
    cfg = AttnConfig(n_layers=6, n_heads=8, n_kv_heads=4, head_dim=256, seq_len=200, rope_theta=1e6,
                     rope_theta_swa=1e4, swa_theta_on_window_layers=1, scale_mode=SCALE_Q_PRESCALED,
                     rope_scale_global=0.125, layer_windows=g.gemma_layer_windows(6, 48, 6), kv_format=KV_BF16)
    for layer in (0, 5):
        check_prefill_then_decode(cfg, m=130, steps=2, seed=layer, layer=layer, chunk=70)


def test_partial_rope_and_adjacent_style():
    cfg = AttnConfig(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=64, rope_dim=32, seq_len=64, kv_format=KV_F32)
    check_prefill_then_decode(cfg, m=40, steps=2, seed=2)
    cfg = AttnConfig(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=64, seq_len=64, rope_style=ROPE_ADJACENT,
                     kv_format=KV_F32)
    check_prefill_then_decode(cfg, m=40, steps=2, seed=3)


def test_adjacent_pairs_over_part_of_a_head_are_rejected():
    """The adjacent-pair rotation of the reference walks the whole head (apply_rope_qk,
    src/engine/runtime/inference.rs:1838-1866); a rope_dim below head_dim with that style is refused at create time,
    so no kernel ever sees it."""
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=64, rope_dim=32, seq_len=64,
                     rope_style=ROPE_ADJACENT, kv_format=KV_F32)
    with pytest.raises(GgrError) as e:
        g.AttnContext(cfg)
    assert "rope_dim" in str(e.value)


def test_position_plan_and_image_block_prefill():
    cfg = AttnConfig(n_layers=1, n_heads=4, n_kv_heads=2, head_dim=64, seq_len=64, rope_theta=1e6,
                     rope_sections=[8, 12, 12, 0], rope_layout=ROPE_INTERLEAVED, image_mode=1,
                     layer_windows=[5], kv_format=KV_F32)
    plan = g.RopePositionPlan()
    plan.append_text(3)
    plan.append_grid([1, 3, 4], 12)
    plan.append_text(4)
    blocks = [(3, 12)]
    ctx, ora = make(cfg, plan=plan, blocks=blocks, prompt_tokens=19)
    rng = np.random.default_rng(9)
    worst = 0.0
    # text chunk, complete image block (staged), text chunk, then decode
    for base, n, block in [(0, 3, False), (3, 12, True), (15, 4, False)]:
        q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
        if block:
            got = ctx.prefill_block(0, base, q, k, v)
        else:
            got = ctx.prefill(0, base, q, k, v)
        want = ora.prefill(0, base, q, k, v, block=block)
        worst = max(worst, float(np.max(np.abs(got - want))))
    for pos in (19, 20):
        q, k, v = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
        worst = max(worst, float(np.max(np.abs(ctx.decode(0, [pos], q, k, v) - ora.decode(0, [pos], q, k, v)))))
    assert worst <= 1e-3
    assert ctx.visible_keys(0, 4) == ora.visible_keys(0, 4) == range(0, 15)
    # a causal chunk may not cut through a bidirectional block (src/engine/runtime/inference.rs:2750-2757)
    with pytest.raises(GgrError):
        ctx.prefill(0, 2, rand(rng, 4, cfg.q_dim), rand(rng, 4, cfg.kv_dim), rand(rng, 4, cfg.kv_dim))


def test_granular_calls_equal_fused_decode():
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=64, seq_len=64, kv_format=KV_Q8_ROW)
    rng = np.random.default_rng(4)
    with g.AttnContext(cfg) as a, g.AttnContext(cfg) as b:
        for pos in range(20):
            q, k, v = rand(rng, cfg.q_dim), rand(rng, cfg.kv_dim), rand(rng, cfg.kv_dim)
            fused = a.decode(0, [pos], q[None], k[None], v[None])[0]
            q2, k2 = q.copy(), k.copy()
            b.apply_rope_qk(0, pos, q2, k2)
            b.kv_write_token(0, pos, k2, v)
            stepwise = b.attention_token(0, pos, q2)
            assert np.max(np.abs(fused - stepwise)) < 1e-6


def test_batched_decode_independent_sequences():
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=4, head_dim=64, seq_len=96, max_batch=5, kv_format=KV_BF16)
    ctx, ora = make(cfg)
    rng = np.random.default_rng(8)
    lens = [10, 37, 64, 1, 90]
    for b, n in enumerate(lens):
        q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
        ctx.prefill(0, 0, q, k, v, seq=b)
        ora.prefill(0, 0, q, k, v, seq=b)
    q, k, v = rand(rng, 5, cfg.q_dim), rand(rng, 5, cfg.kv_dim), rand(rng, 5, cfg.kv_dim)
    got = ctx.decode(0, lens, q, k, v)
    want = ora.decode(0, lens, q, k, v)
    assert np.max(np.abs(got - want)) <= 2e-2


@pytest.mark.parametrize("impl", [IMPL_AUTO, IMPL_SIMT, IMPL_MMA])
@pytest.mark.parametrize("n_heads,n_kv_heads", [(32, 4), (40, 8), (12, 4), (16, 1)])
def test_decode_kernel_families_bf16(impl, n_heads, n_kv_heads):
    cfg = AttnConfig(n_layers=1, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=128, seq_len=1200,
                     rope_theta=1e6, kv_format=KV_BF16, decode_impl=impl)
    check_prefill_then_decode(cfg, m=1100, steps=3, seed=n_heads)


# ---- the benchmark's shapes at sizes the oracle finishes in seconds -------------------------------------

@pytest.mark.parametrize("kv_format", [KV_F32, KV_Q8_ROW])
def test_config1_qwen3_0p6b_decode_T2048(kv_format):
    cfg = presets.qwen3_0p6b_decode(n_layers=1, seq_len=2048, kv_format=kv_format)
    check_prefill_then_decode(cfg, m=2047, steps=1, seed=1001, tol=1e-3)


def test_config2_llama3_prefill_reduced():
    # config 2 at S=1024 (full S=4096 is covered by properties in test_gpu_full_size.py)
    cfg = presets.llama3_8b_prefill(n_layers=1, seq_len=1024)
    rng = np.random.default_rng(1002)
    ctx, ora = make(cfg)
    q, k, v = (bf16_round(rand(rng, 1024, d)) for d in (cfg.q_dim, cfg.kv_dim, cfg.kv_dim))
    import torch
    tq, tk, tv = (torch.from_numpy(x).cuda().to(torch.bfloat16) for x in (q, k, v))
    got = ctx.prefill(0, 0, tq, tk, tv).cpu().numpy()
    want = ora.prefill(0, 0, q, k, v)
    assert np.max(np.abs(got - want)) <= 2e-2


@pytest.mark.parametrize("preset,T", [(presets.qwen3_30b_a3b_decode, 4096), (presets.qwen25_14b_decode, 4096)])
def test_config3_and_5_decode_reduced(preset, T):
    cfg = preset(n_layers=1, seq_len=T, max_batch=2)
    ctx, ora = make(cfg)
    rng = np.random.default_rng(1003)
    for b in range(2):
        n = T - 1 - 100 * b
        q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
        ctx.prefill(0, 0, q, k, v, seq=b)
        ora.prefill(0, 0, q, k, v, seq=b)
    pos = [T - 1, T - 101]
    q, k, v = rand(rng, 2, cfg.q_dim), rand(rng, 2, cfg.kv_dim), rand(rng, 2, cfg.kv_dim)
    assert np.max(np.abs(ctx.decode(0, pos, q, k, v) - ora.decode(0, pos, q, k, v))) <= 2e-2


def test_config4_gemma_chunked_prefill_reduced():
    cfg = presets.gemma3_4b_prefill(n_layers=6, seq_len=768, window=128)
    for layer in (0, 5):
        check_prefill_then_decode(cfg, m=768 - 2, steps=2, seed=1004 + layer, layer=layer, chunk=256)


# ---- KV-sequence sharding: partial states merge to the unsharded result ----------------------------------

@pytest.mark.parametrize("n_ranks", [2, 4])
@pytest.mark.parametrize("window", [0, 100])
def test_sequence_shards_combine_to_unsharded(n_ranks, window):
    T = 512
    base = dict(n_layers=1, n_heads=10, n_kv_heads=2, head_dim=128, seq_len=T, max_batch=3, rope_theta=1e6,
                kv_format=KV_BF16, layer_windows=[window] if window else [])
    full = g.AttnContext(AttnConfig(**base))
    ora = Oracle(AttnConfig(**base), threads=THREADS)
    per = T // n_ranks
    shards = [g.AttnContext(AttnConfig(shard_mode=SHARD_KV_SEQUENCE, shard_pos_begin=r * per, shard_pos_count=per,
                                       n_ranks=n_ranks, rank=r, **base)) for r in range(n_ranks)]
    rng = np.random.default_rng(21)
    lens = [T - 1, 300, 5]
    cfg = full.config
    # fill token by token through decode so every shard appends only the rows it owns
    for step in range(max(lens) + 1):
        pos = [min(step, n) for n in lens]
        live = [b for b, n in enumerate(lens) if step <= n]
        if not live:
            break
        q, k, v = rand(rng, 3, cfg.q_dim), rand(rng, 3, cfg.kv_dim), rand(rng, 3, cfg.kv_dim)
        if step in (5, 300, T - 1):
            want = ora.decode(0, pos, q, k, v)
            got_full = full.decode(0, pos, q, k, v)
            parts = np.stack([s.decode_partial(0, pos, q, k, v) for s in shards])
            got = shards[0].combine_partials(parts)
            for b in live:
                assert np.max(np.abs(got[b] - want[b])) <= 2e-2
                assert np.max(np.abs(got[b] - got_full[b])) <= 5e-3  # bf16 probabilities round differently per split
        else:
            ora.decode(0, pos, q, k, v)
            full.decode(0, pos, q, k, v)
            for s in shards:
                s.decode_partial(0, pos, q, k, v)


# ---- device-pointer mode and error reporting --------------------------------------------------------------

def test_device_pointer_mode_equals_host_mode():
    import torch
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=300, max_batch=2, kv_format=KV_BF16)
    rng = np.random.default_rng(6)
    with g.AttnContext(cfg) as a, g.AttnContext(cfg) as b:
        for seq in range(2):
            q, k, v = rand(rng, 200, cfg.q_dim), rand(rng, 200, cfg.kv_dim), rand(rng, 200, cfg.kv_dim)
            ha = a.prefill(0, 0, q, k, v, seq=seq)
            hb = b.prefill(0, 0, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                           seq=seq)
            torch.cuda.synchronize()
            assert np.array_equal(ha, hb.cpu().numpy())
        q, k, v = rand(rng, 2, cfg.q_dim), rand(rng, 2, cfg.kv_dim), rand(rng, 2, cfg.kv_dim)
        ha = a.decode(0, [200, 200], q, k, v)
        hb = b.decode(0, [200, 200], torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
        torch.cuda.synchronize()
        assert np.array_equal(ha, hb.cpu().numpy())
        assert a.launch_count > 0


def test_invalid_arguments_return_errors():
    for scale in [0.0, -1.0, float("nan"), float("inf")]:
        with pytest.raises(GgrError):
            g.AttnContext(AttnConfig(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=8, seq_len=8,
                                     rope_scale_global=scale))
        with pytest.raises(GgrError):
            g.AttnContext(AttnConfig(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=8, seq_len=8,
                                     rope_scale_local=scale))
    with pytest.raises(GgrError):  # one window entry per layer
        g.AttnContext(AttnConfig(n_layers=2, n_heads=1, n_kv_heads=1, head_dim=8, seq_len=8, layer_windows=[4]))
    cfg = AttnConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=8, seq_len=8)
    with g.AttnContext(cfg) as ctx:
        z = np.zeros((1, 16), np.float32)
        kz = np.zeros((1, 8), np.float32)
        with pytest.raises(GgrError):
            ctx.decode(1, [0], z, kz, kz)  # layer outside the cache
        with pytest.raises(GgrError):
            ctx.decode(0, [8], z, kz, kz)  # position outside the cache
        with pytest.raises(GgrError):
            ctx.decode(0, [0, 1], np.zeros((2, 16), np.float32), np.zeros((2, 8), np.float32),
                       np.zeros((2, 8), np.float32))  # batch above max_batch
        with pytest.raises(GgrError):
            ctx.set_media_blocks([(2, 5), (6, 2)], 12)  # overlapping blocks
        ctx.decode(0, [0], z, kz, kz)  # the context is still usable


# ---- decode fusion: one launch per layer gives the same rows and outputs as rope/append + attention ---------

@pytest.mark.parametrize("kv_format", [KV_F32, KV_BF16, KV_Q8_ROW, KV_Q8_BLOCK32])
@pytest.mark.parametrize("n_heads,n_kv_heads,head_dim", [(8, 4, 64), (32, 4, 128), (4, 4, 32)])
def test_fused_decode_equals_separate_kernels(kv_format, n_heads, n_kv_heads, head_dim):
    import dataclasses
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=700, max_batch=3,
                     rope_theta=1e6, kv_format=kv_format, layer_windows=[0, 300])
    rng = np.random.default_rng(31)
    with g.AttnContext(cfg) as fused, g.AttnContext(dataclasses.replace(cfg, decode_fusion=1)) as plain:
        ora = Oracle(cfg, threads=THREADS)
        lens = [650, 129, 1]
        for b, n in enumerate(lens):
            q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
            for c in (fused, plain):
                c.prefill(1, 0, q, k, v, seq=b)
            ora.prefill(1, 0, q, k, v, seq=b)
        launches_f, launches_p = fused.launch_count, plain.launch_count
        for step in range(3):
            pos = [n + step for n in lens]
            q, k, v = rand(rng, 3, cfg.q_dim), rand(rng, 3, cfg.kv_dim), rand(rng, 3, cfg.kv_dim)
            a = fused.decode(1, pos, q, k, v)
            b_ = plain.decode(1, pos, q, k, v)
            want = ora.decode(1, pos, q, k, v)
            assert np.max(np.abs(a - b_)) <= 1e-5
            assert np.max(np.abs(a - want)) <= TOL[kv_format]
            for s_, p_ in enumerate(pos):
                fk, fv = fused.kv_read_row(1, p_, seq=s_)
                pk, pv = plain.kv_read_row(1, p_, seq=s_)
                assert np.array_equal(fk, pk) and np.array_equal(fv, pv)
        assert fused.launch_count - launches_f == 3       # one launch per step
        assert plain.launch_count - launches_p == 6       # rope/append + attention


# ---- fused shard exchange (peer stores + flags), ranks emulated as contexts of one process -----------------

@pytest.mark.parametrize("n_ranks,n_heads,n_kv_heads", [(2, 10, 2), (4, 8, 8)])
def test_fused_exchange_equals_gather_and_combine(n_ranks, n_heads, n_kv_heads):
    T, B = 600, 3
    base = AttnConfig(n_layers=1, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=128, seq_len=T, max_batch=B,
                      rope_theta=1e6, kv_format=KV_BF16)
    from gguf_runner_b200 import sharding
    ora = Oracle(base, threads=THREADS)
    ranks = [g.AttnContext(sharding.sequence_shard_config(base, r, n_ranks)) for r in range(n_ranks)]
    bufs = [c.exchange_create(B) for c in ranks]
    for c in ranks:
        c.exchange_connect(same_process_ptrs=[b[0] for b in bufs])
    rng = np.random.default_rng(41)
    lens = [T - 3, 310, 7]
    for step in range(max(lens) + 3):
        pos = [min(step, n + 2) for n in lens]
        q, k, v = rand(rng, B, base.q_dim), rand(rng, B, base.kv_dim), rand(rng, B, base.kv_dim)
        want = ora.decode(0, pos, q, k, v)
        # every rank sends (host buffers: each send is complete on return), then every rank receives
        for c in ranks:
            c.exchange_send(0, pos, q, k, v)
        outs = [c.exchange_receive(B, q) for c in ranks]
        if step in (0, 5, 200, 400, max(lens) + 2):
            for o in outs:
                assert np.max(np.abs(o - want)) <= 2e-2, step
            assert all(np.array_equal(outs[0], o) for o in outs[1:])
    for c in ranks:
        c.close()


# ---- pre-attention fixups: Qwen2 biases and per-head RMS QK-norm (qkv_bias_and_norm) ----------------------

@pytest.mark.parametrize("kv_format,with_bias,with_norm", [(KV_F32, True, True), (KV_BF16, False, True),
                                                           (KV_Q8_ROW, True, False), (KV_BF16, True, True)])
def test_bias_and_qk_norm_fixups_match_oracle(kv_format, with_bias, with_norm):
    cfg = AttnConfig(n_layers=2, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=400, rope_theta=1e6, kv_format=kv_format)
    ctx, ora = make(cfg)
    rng = np.random.default_rng(51)
    kw = {}
    if with_bias:
        kw.update(q_bias=rand(rng, cfg.q_dim) * 0.5, k_bias=rand(rng, cfg.kv_dim) * 0.5, v_bias=rand(rng, cfg.kv_dim) * 0.5)
    if with_norm:
        kw.update(q_norm=1.0 + 0.1 * rand(rng, cfg.head_dim), k_norm=1.0 + 0.1 * rand(rng, cfg.head_dim))
    ctx.set_layer_fixups(1, eps=1e-6, **kw)
    ora.set_layer_fixups(1, eps=1e-6, **kw)
    tol = TOL[kv_format]
    q, k, v = rand(rng, 300, cfg.q_dim), rand(rng, 300, cfg.kv_dim), rand(rng, 300, cfg.kv_dim)
    assert np.max(np.abs(ctx.prefill(1, 0, q, k, v) - ora.prefill(1, 0, q, k, v))) <= tol
    for pos in (300, 301):
        q, k, v = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
        assert np.max(np.abs(ctx.decode(1, [pos], q, k, v) - ora.decode(1, [pos], q, k, v))) <= tol
    # a layer without fixups is untouched
    q, k, v = rand(rng, 50, cfg.q_dim), rand(rng, 50, cfg.kv_dim), rand(rng, 50, cfg.kv_dim)
    assert np.max(np.abs(ctx.prefill(0, 0, q, k, v) - ora.prefill(0, 0, q, k, v))) <= tol
    ctx.close()


@pytest.mark.parametrize("head_dim,m,window", [(64, 1400, 0), (128, 1280, 0), (128, 1400, 300)])
def test_prefill_more_work_items_than_sms(head_dim, m, window):
    """Device-pointer prefill with 200-240 query-tile pairs in one launch: the persistent kernel hands items out
    from its work counter, a ragged last pair has no second tile, and the counter must be back at zero for the
    next launch (second layer, then a second chunk on top of the first)."""
    import torch
    cfg = AttnConfig(n_layers=2, n_heads=40, n_kv_heads=8, head_dim=head_dim, seq_len=2048, rope_theta=5e5,
                     kv_format=KV_BF16, layer_windows=[window, window] if window else [])
    rng = np.random.default_rng(m + head_dim)
    ctx, ora = make(cfg)
    worst = 0.0
    for layer in (0, 1):
        pos = 0
        for n in (m, 300):
            q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
            got = ctx.prefill(layer, pos, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                              torch.from_numpy(v).cuda()).cpu().numpy()
            want = ora.prefill(layer, pos, q, k, v)
            worst = max(worst, float(np.max(np.abs(got - want))))
            pos += n
    assert worst <= TOL[KV_BF16], f"max abs err {worst}"
    ctx.close()


# ---- TurboQuant cache (src/engine/runtime/inference.rs:885-982, :1246-1334) ----

@pytest.mark.parametrize("head_dim,n_heads,n_kv_heads,style", [(64, 4, 2, ROPE_NEOX), (128, 8, 2, ROPE_ADJACENT),
                                                                (256, 4, 4, ROPE_NEOX)])
def test_turboquant_append_is_bit_exact(head_dim, n_heads, n_kv_heads, style):
    """Codes, sign bits, sigma and residual norm of appended rows equal the oracle's bit for bit wherever the inputs
    are bit-identical: every V row, and the K row of the granular write (already rotated keys). A zero row takes the
    sigma == 0 arm."""
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=64, rope_theta=1e6,
                     rope_style=style, kv_format=KV_TURBO)
    rng = np.random.default_rng(head_dim)
    ctx, ora = make(cfg)
    m = 20
    q, k, v = rand(rng, m, cfg.q_dim), rand(rng, m, cfg.kv_dim), rand(rng, m, cfg.kv_dim)
    k[3] = 0.0
    v[5] = 0.0
    ctx.prefill(1, 0, q, k, v)
    ora.prefill(1, 0, q, k, v)
    q1, k1, v1 = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
    ctx.decode(1, [m], q1, k1, v1)
    ora.decode(1, [m], q1, k1, v1)
    kr = rand(rng, cfg.kv_dim)
    ctx.kv_write_token(1, m + 1, kr, v1[0])
    ora.kv_write_token(1, m + 1, kr, v1[0])
    for pos in range(m + 2):
        got, want = ctx.kv_read_turbo(1, pos), ora.kv_read_turbo(1, pos)
        for name in want:
            if name.startswith("v_") or pos == m + 1:
                assert np.array_equal(got[name], want[name]), (pos, name)
        # keys written through prefill / decode were rotated on the device, whose sincosf may differ from the host's
        # cosf / sinf in the last bit: norms agree to rounding and at most a few elements sit on the other side
        # of a threshold
        np.testing.assert_allclose(got["k_scale"], want["k_scale"], rtol=2e-6)
        np.testing.assert_allclose(got["k_rnorm"], want["k_rnorm"], rtol=2e-5)
        flipped = np.unpackbits(got["k_base"] ^ want["k_base"]).sum() + np.unpackbits(got["k_sign"] ^ want["k_sign"]).sum()
        assert flipped <= 4, (pos, int(flipped))
    ctx.close()


@pytest.mark.parametrize("head_dim,n_heads,n_kv_heads", [(64, 8, 2), (128, 8, 8), (128, 12, 4), (256, 4, 2)])
@pytest.mark.parametrize("window", [0, 24])
@pytest.mark.parametrize("impl", [IMPL_AUTO, IMPL_SIMT])
def test_turboquant_prefill_and_decode_match_oracle(head_dim, n_heads, n_kv_heads, window, impl):
    """Prefill rows and CUDA-core decode compute in f32 (1e-3); head_dim 128 decode runs on the tensor cores by
    default, with bf16 queries, centroids and probabilities (the bf16 tolerance, 2e-2)."""
    cfg = AttnConfig(n_layers=1, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=400, rope_theta=1e6,
                     rope_style=ROPE_NEOX, kv_format=KV_TURBO, layer_windows=[window] if window else [],
                     decode_impl=impl)
    tol = TOL[KV_BF16] if (head_dim == 128 and impl == IMPL_AUTO) else TOL[KV_TURBO]
    check_prefill_then_decode(cfg, m=150, steps=3, seed=head_dim + window, chunk=64, tol=tol)


def test_turboquant_long_decode_uses_splits_and_batches():
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=3000, max_batch=3, rope_theta=1e6,
                     rope_style=ROPE_NEOX, kv_format=KV_TURBO)
    rng = np.random.default_rng(5)
    ctx, ora = make(cfg)
    for seq, n in enumerate((2500, 1200, 40)):
        q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
        ctx.prefill(0, 0, q, k, v, seq=seq)
        ora.prefill(0, 0, q, k, v, seq=seq)
    q, k, v = rand(rng, 3, cfg.q_dim), rand(rng, 3, cfg.kv_dim), rand(rng, 3, cfg.kv_dim)
    got = ctx.decode(0, [2500, 1200, 40], q, k, v)
    want = ora.decode(0, [2500, 1200, 40], q, k, v)
    assert ctx.last_split_count > 1
    err = float(np.max(np.abs(got - want)))
    assert err <= TOL[KV_BF16], err  # tensor-core decode: bf16 queries, centroids and probabilities
    ctx.close()


def test_turboquant_tensor_core_decode_at_full_grouping():
    """16 query heads per KV head (all rows of the MMA tile in use), a key range that is no multiple of the tile,
    several sequences with different lengths; compared with the oracle and with the CUDA-core kernel."""
    base = dict(n_layers=1, n_heads=32, n_kv_heads=2, head_dim=128, seq_len=1500, max_batch=2, rope_theta=1e6,
                rope_style=ROPE_NEOX, kv_format=KV_TURBO)
    rng = np.random.default_rng(9)
    lens = (1237, 333)
    ctx, ora = make(AttnConfig(**base))
    ref = g.AttnContext(AttnConfig(decode_impl=IMPL_SIMT, **base))
    for seq, n in enumerate(lens):
        q, k, v = rand(rng, n, 32 * 128), rand(rng, n, 256), rand(rng, n, 256)
        for c in (ctx, ref):
            c.prefill(0, 0, q, k, v, seq=seq)
        ora.prefill(0, 0, q, k, v, seq=seq)
    q, k, v = rand(rng, 2, 32 * 128), rand(rng, 2, 256), rand(rng, 2, 256)
    got = ctx.decode(0, list(lens), q, k, v)
    exact = ref.decode(0, list(lens), q, k, v)
    want = ora.decode(0, list(lens), q, k, v)
    assert np.max(np.abs(exact - want)) <= TOL[KV_TURBO]
    assert np.max(np.abs(got - want)) <= TOL[KV_BF16]
    ctx.close()
    ref.close()


def test_turboquant_prefill_on_tensor_cores_is_opt_in():
    """prefill_impl = MMA sends TurboQuant prefill rows through the tensor-core kernel (bf16 tolerance); the default
    keeps them on the f32 kernel (1e-3)."""
    base = dict(n_layers=1, n_heads=16, n_kv_heads=4, head_dim=128, seq_len=600, rope_theta=1e6, rope_style=ROPE_NEOX,
                kv_format=KV_TURBO)
    rng = np.random.default_rng(21)
    q, k, v = rand(rng, 500, 16 * 128), rand(rng, 500, 512), rand(rng, 500, 512)
    want = Oracle(AttnConfig(**base), threads=THREADS).prefill(0, 0, q, k, v)
    exact = g.AttnContext(AttnConfig(**base))
    fast = g.AttnContext(AttnConfig(prefill_impl=IMPL_MMA, **base))
    assert np.max(np.abs(exact.prefill(0, 0, q, k, v) - want)) <= TOL[KV_TURBO]
    assert np.max(np.abs(fast.prefill(0, 0, q, k, v) - want)) <= TOL[KV_BF16]
    exact.close()
    fast.close()
