"""KV-head sharding: one context per rank holding a contiguous group of KV heads and their query heads.

Attention is independent per KV head (the reference fans heads out and reads kv_head = h / kv_mul,
src/engine/runtime/inference.rs:2002-2019), so head-sharded contexts need no collective: rank r's output
is the slice of q_dim it owns. Here the ranks are contexts on one GPU; their outputs and cache rows must
reproduce the unsharded context's slices and the oracle's.
"""
import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200 import sharding
from gguf_runner_b200.binding import AttnConfig, KV_BF16, KV_F32, KV_Q8_BLOCK32, KV_Q8_ROW
from tests.oracle_binding import Oracle

pytestmark = pytest.mark.gpu
THREADS = 8
TOL = {KV_F32: 1e-3, KV_Q8_ROW: 1e-3, KV_Q8_BLOCK32: 1e-3, KV_BF16: 2e-2}


def rand(rng, *shape):
    return rng.standard_normal(shape).astype(np.float32)


@pytest.mark.parametrize("kv_format", [KV_BF16, KV_F32, KV_Q8_BLOCK32])
@pytest.mark.parametrize("n_ranks,n_heads,n_kv_heads", [(2, 32, 4), (4, 32, 4), (4, 16, 8)])
def test_head_shards_reproduce_unsharded_slices(kv_format, n_ranks, n_heads, n_kv_heads):
    B, m = 3, 333
    base = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=128, seq_len=512, max_batch=B,
                      rope_theta=1e6, kv_format=kv_format, layer_windows=[0, 100])
    full = g.AttnContext(base)
    ora = Oracle(base, threads=THREADS)
    plans = [sharding.head_shard_config(base, r, n_ranks) for r in range(n_ranks)]
    ranks = [g.AttnContext(p[0]) for p in plans]
    rng = np.random.default_rng(n_ranks * 100 + n_heads)
    tol = TOL[kv_format]
    for layer in (0, 1):
        lens = [m, 200, 17]
        for b, n in enumerate(lens):
            q, k, v = rand(rng, n, base.q_dim), rand(rng, n, base.kv_dim), rand(rng, n, base.kv_dim)
            want = ora.prefill(layer, 0, q, k, v, seq=b)
            got_full = full.prefill(layer, 0, q, k, v, seq=b)
            assert np.max(np.abs(got_full - want)) <= tol
            for ctx, (_cfg, qs, ks) in zip(ranks, plans):
                got = ctx.prefill(layer, 0, np.ascontiguousarray(q[:, qs]), np.ascontiguousarray(k[:, ks]),
                                  np.ascontiguousarray(v[:, ks]), seq=b)
                assert np.max(np.abs(got - want[:, qs])) <= tol
                assert np.max(np.abs(got - got_full[:, qs])) <= tol / 4
        for step in range(2):
            pos = [n + step for n in lens]
            q, k, v = rand(rng, B, base.q_dim), rand(rng, B, base.kv_dim), rand(rng, B, base.kv_dim)
            want = ora.decode(layer, pos, q, k, v)
            got_full = full.decode(layer, pos, q, k, v)
            assert np.max(np.abs(got_full - want)) <= tol
            for ctx, (_cfg, qs, ks) in zip(ranks, plans):
                got = ctx.decode(layer, pos, np.ascontiguousarray(q[:, qs]), np.ascontiguousarray(k[:, ks]),
                                 np.ascontiguousarray(v[:, ks]))
                assert np.max(np.abs(got - want[:, qs])) <= tol
        # cache rows: every element is produced by the same arithmetic in both layouts
        for b, row in [(0, 0), (0, m), (1, 199), (2, 18)]:
            fk, fv = full.kv_read_row(layer, row, seq=b)
            for ctx, (_cfg, _qs, ks) in zip(ranks, plans):
                sk, sv = ctx.kv_read_row(layer, row, seq=b)
                assert np.array_equal(sk, fk[ks]) and np.array_equal(sv, fv[ks])
    for c in [full] + ranks:
        c.close()


def test_head_shards_with_row_scaled_q8_cache_follow_their_own_rows():
    """The q8 row format keeps one scale per cache row over all the KV heads a context holds
    (src/engine/runtime/inference.rs:1906-1916); a head shard therefore quantises with the maximum over its own
    heads and is compared with an oracle that holds the same heads."""
    base = AttnConfig(n_layers=1, n_heads=16, n_kv_heads=4, head_dim=128, seq_len=256, rope_theta=1e6,
                      kv_format=KV_Q8_ROW)
    rng = np.random.default_rng(5)
    q, k, v = rand(rng, 150, base.q_dim), rand(rng, 150, base.kv_dim), rand(rng, 150, base.kv_dim)
    for r in range(2):
        cfg, qs, ks = sharding.head_shard_config(base, r, 2)
        ora = Oracle(cfg, threads=THREADS)
        with g.AttnContext(cfg) as ctx:
            ql, kl, vl = (np.ascontiguousarray(x) for x in (q[:, qs], k[:, ks], v[:, ks]))
            assert np.max(np.abs(ctx.prefill(0, 0, ql, kl, vl) - ora.prefill(0, 0, ql, kl, vl))) <= 1e-3
            kq, vq, ksc, vsc = ctx.kv_export(0, 0, 150)
            for row in (0, 77, 149):
                okq, ovq, oks, ovs = ora.kv_read_q8(0, row)
                assert np.array_equal(kq[row], okq) and np.array_equal(vq[row], ovq)
                assert ksc[row] == oks[0] and vsc[row] == ovs[0]
