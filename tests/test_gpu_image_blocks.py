"""Bidirectional image blocks on the tensor-core (tcgen05) prefill kernels.

The reference evaluates a complete image block in two passes (stage every row's K / V, then attend
every row with block-wide visibility: src/engine/runtime/media_prefill.rs:84-119,
src/engine/runtime/attention.rs:87-94). The bf16 cache at head_dim 64 / 128 / 256 is what sends
ggr_attn_prefill_block to the tcgen05 kernels, whose per-tile key ranges are derived from a tile's
first and last row: these cases put blocks across 128-row query-tile borders and 128-key tile
borders, with windows shorter than the blocks, after a text prefix, and follow them with a text
chunk and decode steps. Tolerance 2e-2 (bf16 operands).
"""
import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import AttnConfig, GgrError, IMAGE_BIDIRECTIONAL, IMPL_TCGEN05, KV_BF16, SCALE_Q_PRESCALED
from tests.oracle_binding import Oracle

pytestmark = pytest.mark.gpu
THREADS = 8


def rand(rng, *shape):
    return rng.standard_normal(shape).astype(np.float32)


# (prompt layout) text [0, 100), block [100, 160) across the row-128 border, text [160, 420),
# block [420, 620) across the key-512 border and two query tiles, text [620, 660)
BLOCKS = [(100, 60), (420, 200)]
SEGMENTS = [(0, 100, False), (100, 60, True), (160, 260, False), (420, 200, True), (620, 40, False)]
PROMPT = 660


@pytest.mark.parametrize("head_dim,n_heads,n_kv_heads", [(128, 4, 2), (256, 4, 2), (64, 4, 1)])
@pytest.mark.parametrize("windows", [(0, 0), (32, 0), (150, 300)])
def test_image_blocks_on_tensor_core_prefill(head_dim, n_heads, n_kv_heads, windows):
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=768,
                     rope_theta=1e6, kv_format=KV_BF16, image_mode=IMAGE_BIDIRECTIONAL,
                     layer_windows=list(windows) if any(windows) else [], prefill_impl=IMPL_TCGEN05,
                     scale_mode=SCALE_Q_PRESCALED if head_dim == 256 else 0)
    ctx = g.AttnContext(cfg)
    ora = Oracle(cfg, threads=THREADS)
    ctx.set_media_blocks(BLOCKS, PROMPT)
    ora.set_media_blocks(BLOCKS, PROMPT)
    rng = np.random.default_rng(head_dim + sum(windows))
    worst = 0.0
    for layer in (0, 1):
        for base, n, block in SEGMENTS:
            q, k, v = rand(rng, n, cfg.q_dim), rand(rng, n, cfg.kv_dim), rand(rng, n, cfg.kv_dim)
            got = (ctx.prefill_block if block else ctx.prefill)(layer, base, q, k, v)
            want = ora.prefill(layer, base, q, k, v, block=block)
            err = float(np.max(np.abs(got - want)))
            assert err <= 2e-2, (layer, base, n, block, err)
            worst = max(worst, err)
        for pos in (PROMPT, PROMPT + 1):
            q, k, v = rand(rng, 1, cfg.q_dim), rand(rng, 1, cfg.kv_dim), rand(rng, 1, cfg.kv_dim)
            err = float(np.max(np.abs(ctx.decode(layer, [pos], q, k, v) - ora.decode(layer, [pos], q, k, v))))
            assert err <= 2e-2, (layer, pos, err)
    # rows inside a block see the whole block, also past a window; rows after it are causal again
    assert ctx.visible_keys(0, 430) == ora.visible_keys(0, 430)
    assert ctx.visible_keys(0, 430).stop == 620
    assert ctx.visible_keys(1, 619) == ora.visible_keys(1, 619)
    # a causal chunk may not cut a block, a staged call must cover whole blocks
    with pytest.raises(GgrError):
        ctx.prefill(0, 90, rand(rng, 20, cfg.q_dim), rand(rng, 20, cfg.kv_dim), rand(rng, 20, cfg.kv_dim))
    with pytest.raises(GgrError):
        ctx.prefill_block(0, 100, rand(rng, 30, cfg.q_dim), rand(rng, 30, cfg.kv_dim), rand(rng, 30, cfg.kv_dim))
    ctx.close()


def test_block_spanning_several_tiles_with_text_in_the_same_staged_call():
    """One staged call may carry text rows around a block (the reference stages whole spans); the block here
    covers rows 130..519 of a 600-row call at base 256, so tiles hold block rows, text rows, or both."""
    cfg = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=128, seq_len=1024, rope_theta=1e6,
                     kv_format=KV_BF16, image_mode=IMAGE_BIDIRECTIONAL, layer_windows=[200],
                     prefill_impl=IMPL_TCGEN05)
    blocks = [(256 + 130, 390)]
    ctx = g.AttnContext(cfg)
    ora = Oracle(cfg, threads=THREADS)
    ctx.set_media_blocks(blocks, 900)
    ora.set_media_blocks(blocks, 900)
    rng = np.random.default_rng(77)
    q, k, v = rand(rng, 256, cfg.q_dim), rand(rng, 256, cfg.kv_dim), rand(rng, 256, cfg.kv_dim)
    assert np.max(np.abs(ctx.prefill(0, 0, q, k, v) - ora.prefill(0, 0, q, k, v))) <= 2e-2
    q, k, v = rand(rng, 600, cfg.q_dim), rand(rng, 600, cfg.kv_dim), rand(rng, 600, cfg.kv_dim)
    got = ctx.prefill_block(0, 256, q, k, v)
    want = ora.prefill(0, 256, q, k, v, block=True)
    assert np.max(np.abs(got - want)) <= 2e-2
    ctx.close()
