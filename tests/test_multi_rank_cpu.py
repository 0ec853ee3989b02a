"""The multi-rank protocol of KV-sequence sharding, run as two gloo ranks on the CPU.

Each rank holds a slab of positions, computes the partial softmax state (o / l, m, l) of its slab
(here with numpy over rows the oracle stored), all-gathers the partials and merges them with the
same formula the device merge uses. The result must equal the oracle's attention over the whole
cache. The device kernels themselves are covered by the GPU tests.
"""
import math
import os
import socket

import numpy as np
import pytest

from gguf_runner_b200 import sharding
from gguf_runner_b200.binding import AttnConfig, KV_F32


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial_state(K, V, q, G, scale_log2):
    """(o / l, m, l) per head over the rows K, V ([T][Hkv][D]) for rotated q ([H][D])."""
    H, D = q.shape
    out = np.zeros((H, D + 2), np.float32)
    for h in range(H):
        if K.shape[0] == 0:
            out[h, D] = -np.inf
            continue
        s = (K[:, h // G, :].astype(np.float64) @ q[h].astype(np.float64)) * scale_log2
        m = s.max()
        p = np.exp2(s - m)
        l = p.sum()
        out[h, :D] = (p @ V[:, h // G, :].astype(np.float64)) / l
        out[h, D] = m
        out[h, D + 1] = l
    return out


def _worker(rank, world, port, q_out):
    import torch.distributed as dist
    from tests.oracle_binding import Oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    T, window = 97, 40
    results = []
    for layer_windows in ([], [window]):
        cfg = AttnConfig(n_layers=1, n_heads=6, n_kv_heads=2, head_dim=16, seq_len=T, rope_theta=1e4, kv_format=KV_F32,
                         layer_windows=layer_windows)
        rng = np.random.default_rng(5)  # same inputs on every rank (q, k, v are replicated)
        ora = Oracle(cfg)
        q = rng.standard_normal((T, cfg.q_dim)).astype(np.float32)
        k = rng.standard_normal((T, cfg.kv_dim)).astype(np.float32)
        v = rng.standard_normal((T, cfg.kv_dim)).astype(np.float32)
        want = ora.prefill(0, 0, q, k, v)
        begin, count = sharding.sequence_slabs(T, world)[rank]
        rows = [ora.kv_read_row(0, t) for t in range(T)]
        K = np.stack([r[0] for r in rows]).reshape(T, 2, 16)
        V = np.stack([r[1] for r in rows]).reshape(T, 2, 16)
        worst = 0.0
        for pos in (0, 10, 48, 49, 96):
            qr, kr = q[pos].copy(), k[pos].copy()
            ora.apply_rope_qk(0, pos, qr, kr)
            vis = ora.visible_keys(0, pos)
            lo, hi = max(vis.start, begin), min(vis.stop, begin + count)
            sl = slice(lo, max(lo, hi))
            part = _partial_state(K[sl], V[sl], qr.reshape(6, 16), 3, math.log2(math.e) / 4.0)
            gathered = [torch.zeros(6, 18) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(part))
            parts = np.stack([g.numpy() for g in gathered])[:, None]
            got = sharding.merge_partials(parts)[0]
            worst = max(worst, float(np.max(np.abs(got - want[pos]))))
            assert sharding.owner_of(pos, T, world) == (0 if pos < sharding.sequence_slabs(T, world)[0][1] else 1)
        results.append(worst)
    if rank == 0:
        q_out.put(results)
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_shards_merge_over_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = q_out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert max(results) < 1e-5, results


def test_slab_and_head_plans():
    assert sharding.sequence_slabs(10, 3) == [(0, 4), (4, 3), (7, 3)]
    assert sharding.sequence_slabs(131072, 8)[7] == (114688, 16384)
    with pytest.raises(ValueError):
        sharding.sequence_slabs(2, 3)
    cfg = AttnConfig(n_layers=1, n_heads=32, n_kv_heads=4, head_dim=128, seq_len=64)
    local, qs, ks = sharding.head_shard_config(cfg, 1, 4)
    assert (local.n_heads, local.n_kv_heads) == (8, 1)
    assert (qs.start, qs.stop, ks.start, ks.stop) == (1024, 2048, 128, 256)
    with pytest.raises(ValueError):
        sharding.head_shard_config(cfg, 0, 3)
    s = sharding.sequence_shard_config(cfg, 1, 2)
    assert (s.shard_mode, s.shard_pos_begin, s.shard_pos_count) == (2, 32, 32)


def test_merge_partials_ignores_empty_ranks():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((1, 2, 3, 10)).astype(np.float32)
    a[..., -1] = np.abs(a[..., -1]) + 0.1
    empty = np.zeros_like(a)
    empty[..., -2] = -np.inf
    merged = sharding.merge_partials(np.concatenate([a, empty]))
    assert np.allclose(merged, a[0, ..., :-2].reshape(2, -1), atol=1e-6)
