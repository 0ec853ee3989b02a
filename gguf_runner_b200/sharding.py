"""Host-side plans for running the attention path on several GPUs of one box.

Two ways the path shards (the reference itself is single process):
  * KV-head sharding: rank r owns a contiguous group of KV heads and their query heads; outputs are
    disjoint slices of q_dim, so attention needs no collective.
  * KV-sequence sharding: rank r holds a contiguous slab of cache positions; every rank attends over
    its slab and the per-rank partial softmax states (o / l, m, l) are all-gathered and merged.
"""
from __future__ import annotations

import dataclasses
from typing import List, Tuple

import numpy as np

from .binding import AttnConfig, SHARD_KV_SEQUENCE


def sequence_slabs(seq_len: int, n_ranks: int) -> List[Tuple[int, int]]:
    """(begin, count) of the positions each rank holds: contiguous, covering [0, seq_len), sizes differ by at most 1."""
    if n_ranks <= 0 or seq_len < n_ranks:
        raise ValueError("need at least one position per rank")
    base, extra = divmod(seq_len, n_ranks)
    slabs, begin = [], 0
    for r in range(n_ranks):
        count = base + (1 if r < extra else 0)
        slabs.append((begin, count))
        begin += count
    return slabs


def sequence_shard_config(cfg: AttnConfig, rank: int, n_ranks: int) -> AttnConfig:
    begin, count = sequence_slabs(cfg.seq_len, n_ranks)[rank]
    return dataclasses.replace(cfg, shard_mode=SHARD_KV_SEQUENCE, shard_pos_begin=begin, shard_pos_count=count,
                               n_ranks=n_ranks, rank=rank)


def owner_of(pos: int, seq_len: int, n_ranks: int) -> int:
    """Rank whose slab holds `pos` (the rank that appends the new row)."""
    for r, (begin, count) in enumerate(sequence_slabs(seq_len, n_ranks)):
        if begin <= pos < begin + count:
            return r
    raise ValueError("position outside the cache")


def head_shard_config(cfg: AttnConfig, rank: int, n_ranks: int) -> Tuple[AttnConfig, slice, slice]:
    """Config of rank r under KV-head sharding plus the slices of q_dim and kv_dim it owns."""
    if cfg.n_kv_heads % n_ranks != 0:
        raise ValueError("n_kv_heads must be divisible by the number of ranks")
    hkv = cfg.n_kv_heads // n_ranks
    g = cfg.n_heads // cfg.n_kv_heads
    local = dataclasses.replace(cfg, n_heads=hkv * g, n_kv_heads=hkv, n_ranks=n_ranks, rank=rank)
    d = cfg.head_dim
    return local, slice(rank * hkv * g * d, (rank + 1) * hkv * g * d), slice(rank * hkv * d, (rank + 1) * hkv * d)


def merge_partials(parts: np.ndarray) -> np.ndarray:
    """Host statement of the merge ggr_attn_combine_partials performs: parts is [n][B][H][D+2] holding
    (o / l, m in base-2 units, l); returns [B][H*D]."""
    parts = np.asarray(parts, dtype=np.float64)
    o, m, l = parts[..., :-2], parts[..., -2], parts[..., -1]
    m_star = np.max(m, axis=0)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isneginf(m), 0.0, l * np.exp2(m - m_star))
    den = np.sum(w, axis=0)
    num = np.sum(w[..., None] * o, axis=0)
    out = np.where(den[..., None] > 0, num / np.where(den[..., None] > 0, den[..., None], 1.0), 0.0)
    return out.reshape(out.shape[0], -1).astype(np.float32)
