"""The bounded wait of the fused shard exchange running out, and recovery from it.

Failure is made on the host: a rank that never sends. The waiting kernel gives up after the configured bound
(exchange_wait_us), stores an error status and returns; the host reads GGR_ERR_TIMEOUT and the context stays
usable. Nothing here faults, traps or spins without a limit. The ranks are contexts on one GPU, and every
send is complete before a receive is issued (a waiting kernel never depends on a co-scheduled producer).
"""
import dataclasses
import time

import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200 import sharding
from gguf_runner_b200.binding import AttnConfig, GgrError, KV_BF16
from tests.oracle_binding import Oracle

pytestmark = pytest.mark.gpu

GGR_ERR_TIMEOUT, GGR_ERR_COMM = 6, 7


def rand(rng, *shape):
    return rng.standard_normal(shape).astype(np.float32)


def make_ranks(base, n_ranks, wait_us):
    ranks = [g.AttnContext(dataclasses.replace(sharding.sequence_shard_config(base, r, n_ranks), exchange_wait_us=wait_us))
             for r in range(n_ranks)]
    bufs = [c.exchange_create(base.max_batch) for c in ranks]
    for c in ranks:
        c.exchange_connect(same_process_ptrs=[b[0] for b in bufs])
    return ranks


def test_receive_times_out_when_a_rank_never_sends_and_the_next_step_still_works():
    T, B = 256, 2
    base = AttnConfig(n_layers=1, n_heads=10, n_kv_heads=2, head_dim=128, seq_len=T, max_batch=B, rope_theta=1e6,
                      kv_format=KV_BF16)
    ora = Oracle(base, threads=4)
    ranks = make_ranks(base, 2, wait_us=2000)
    rng = np.random.default_rng(3)
    # a few complete steps first
    for step in range(3):
        pos = [step, step]
        q, k, v = rand(rng, B, base.q_dim), rand(rng, B, base.kv_dim), rand(rng, B, base.kv_dim)
        want = ora.decode(0, pos, q, k, v)
        for c in ranks:
            c.exchange_send(0, pos, q, k, v)
        for c in ranks:
            assert np.max(np.abs(c.exchange_receive(B, q) - want)) <= 2e-2
    # rank 1 never joins this step: rank 0's wait runs out within its bound and reports a status
    pos = [3, 3]
    q, k, v = rand(rng, B, base.q_dim), rand(rng, B, base.kv_dim), rand(rng, B, base.kv_dim)
    ranks[0].exchange_send(0, pos, q, k, v)
    t0 = time.perf_counter()
    with pytest.raises(GgrError) as e:
        ranks[0].exchange_receive(B, q)
    assert e.value.status == GGR_ERR_TIMEOUT
    assert time.perf_counter() - t0 < 1.0
    # the error word is cleared with the report: the context synchronises cleanly afterwards
    ranks[0].synchronize()
    assert ranks[0].exchange_epoch == 4 and ranks[1].exchange_epoch == 3
    # the ranks agree on the largest step counter on the host and repeat the step (an append is idempotent)
    top = max(c.exchange_epoch for c in ranks)
    for c in ranks:
        c.exchange_resync(top)
    want = ora.decode(0, pos, q, k, v)
    for c in ranks:
        c.exchange_send(0, pos, q, k, v)
    outs = [c.exchange_receive(B, q) for c in ranks]
    for o in outs:
        assert np.max(np.abs(o - want)) <= 2e-2
    assert np.array_equal(outs[0], outs[1])
    for c in ranks:
        c.close()


def test_a_rank_that_fell_behind_is_told_instead_of_merging_stale_states():
    T, B = 128, 1
    base = AttnConfig(n_layers=1, n_heads=8, n_kv_heads=2, head_dim=64, seq_len=T, max_batch=B, rope_theta=1e6,
                      kv_format=KV_BF16)
    ora = Oracle(base, threads=2)
    ranks = make_ranks(base, 2, wait_us=2000)
    rng = np.random.default_rng(4)
    q, k, v = rand(rng, B, base.q_dim), rand(rng, B, base.kv_dim), rand(rng, B, base.kv_dim)
    # rank 0 runs three sends ahead (its receives in between time out; the test ignores them)
    for _ in range(3):
        ranks[0].exchange_send(0, [0], q, k, v)
    ranks[1].exchange_send(0, [0], q, k, v)
    with pytest.raises(GgrError) as e:
        ranks[1].exchange_receive(B, q)   # its step 1 finds rank 0's flag at 3
    assert e.value.status == GGR_ERR_COMM
    # one step ahead is legitimate (the peer finished this step and sent the next into the other parity)
    top = max(c.exchange_epoch for c in ranks)
    for c in ranks:
        c.exchange_resync(top)
    want = ora.decode(0, [0], q, k, v)
    for c in ranks:
        c.exchange_send(0, [0], q, k, v)
    ranks[0].exchange_send(0, [0], q, k, v)           # rank 0 already in the next step
    got = ranks[1].exchange_receive(B, q)
    assert np.max(np.abs(got - want)) <= 2e-2
    with pytest.raises(GgrError):
        ranks[0].exchange_resync(0)                    # the counter only moves forward
    for c in ranks:
        c.close()


def test_wait_bound_is_validated():
    with pytest.raises(GgrError):
        g.AttnContext(AttnConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=64, seq_len=16, exchange_wait_us=-5))
