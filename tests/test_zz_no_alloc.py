"""The allocation-free attention entry point against the regular one.

Hosts that cannot call cudaMalloc while decoding (all of HBM already handed to
caches and weights, or a token loop that must not take an allocation's
device-wide synchronisation) use ggr_attn_attention_tokens_static, whose
split-KV scratch is a fixed array inside the library. This test calls it
through the C ABI twice in a row (the second call finds the first call's data
in the shared array) and compares with ggr_attn_attention_token, which uses
scratch grown with cudaMalloc. Collected last on purpose: a run that stops at
the first failure has then already run every other test.
"""
import numpy as np
import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import AttnConfig, GgrError, KV_BF16, KV_F32, KV_Q8_BLOCK32, KV_Q8_ROW
from tests.oracle_binding import Oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_format,n_heads,n_kv_heads,head_dim,window",
                         [(KV_BF16, 16, 2, 128, 0), (KV_Q8_ROW, 4, 2, 128, 0), (KV_F32, 4, 2, 64, 0),
                          (KV_Q8_BLOCK32, 8, 2, 64, 500), (KV_BF16, 10, 2, 128, 1200)])
def test_static_scratch_entry_matches_regular_entry(kv_format, n_heads, n_kv_heads, head_dim, window):
    import torch
    B, T = 3, 3000
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, seq_len=T, max_batch=B,
                     rope_theta=1e6, kv_format=kv_format, layer_windows=[0, window] if window else [])
    rng = np.random.default_rng(17)
    ora = Oracle(cfg, threads=8)
    with g.AttnContext(cfg) as ctx:
        lens = [T - 1, 2000, 700]
        for b, n in enumerate(lens):
            q = rng.standard_normal((n, cfg.q_dim)).astype(np.float32)
            k = rng.standard_normal((n, cfg.kv_dim)).astype(np.float32)
            v = rng.standard_normal((n, cfg.kv_dim)).astype(np.float32)
            ctx.prefill(1, 0, q, k, v, seq=b)
            if b == 2:
                ora.prefill(1, 0, q, k, v, seq=b)  # the shortest sequence also goes through the oracle
        pos = [n - 1 for n in lens]
        launches = ctx.launch_count
        for call in range(2):
            q = rng.standard_normal((B, cfg.q_dim)).astype(np.float32)
            want = np.stack([ctx.attention_token(1, pos[b], q[b], seq=b) for b in range(B)])
            tq = torch.from_numpy(q).cuda()
            got = ctx.attention_tokens_static(1, pos, tq)
            torch.cuda.synchronize()
            # same kernels and split rule on the same data; only the split count may differ with the
            # batch, so allow summation-order noise (the suite's f32 tolerance is 1e-3, bf16 2e-2)
            tol = 2e-2 if kv_format == KV_BF16 else 1e-3
            err = float(np.max(np.abs(got.cpu().numpy() - want)))
            assert err <= tol, (call, err)
            assert err <= 5e-3
            # and against the CPU oracle on the sequence it holds (q is already rotated: attention only)
            want_cpu = ora.attention_token(1, pos[2], q[2], seq=2)
            assert float(np.max(np.abs(got.cpu().numpy()[2] - want_cpu))) <= tol
        assert ctx.launch_count > launches


def test_static_scratch_is_shared_by_contexts_on_one_stream():
    """Two contexts alternate on one stream; each call finds the other's data in the array."""
    import torch
    T = 2500
    cfgs = [AttnConfig(n_layers=1, n_heads=16, n_kv_heads=2, head_dim=128, seq_len=T, rope_theta=1e6, kv_format=KV_BF16),
            AttnConfig(n_layers=1, n_heads=4, n_kv_heads=4, head_dim=64, seq_len=T, rope_theta=1e6, kv_format=KV_F32)]
    rng = np.random.default_rng(23)
    ctxs = [g.AttnContext(c) for c in cfgs]
    stream = torch.cuda.current_stream().cuda_stream or 1
    for ctx, cfg in zip(ctxs, cfgs):
        q = rng.standard_normal((T - 1, cfg.q_dim)).astype(np.float32)
        k = rng.standard_normal((T - 1, cfg.kv_dim)).astype(np.float32)
        v = rng.standard_normal((T - 1, cfg.kv_dim)).astype(np.float32)
        ctx.prefill(0, 0, q, k, v)
        ctx.set_stream(stream)
    for call in range(4):
        ctx, cfg = ctxs[call & 1], cfgs[call & 1]
        q = rng.standard_normal((1, cfg.q_dim)).astype(np.float32)
        want = ctx.attention_token(0, T - 2, q[0])
        got = ctx.attention_tokens_static(0, [T - 2], torch.from_numpy(q).cuda())
        torch.cuda.synchronize()
        assert ctx.last_split_count > 1
        assert float(np.max(np.abs(got.cpu().numpy()[0] - want))) <= 5e-3
    for ctx in ctxs:
        ctx.close()


def test_static_scratch_entry_rejects_oversized_calls():
    import torch
    # a split call needs 2 * B * n_heads * (head_dim + 2) floats in the built-in 8 MiB array
    cfg = AttnConfig(n_layers=1, n_heads=128, n_kv_heads=1, head_dim=256, seq_len=4096, max_batch=32,
                     kv_format=KV_BF16)
    with g.AttnContext(cfg) as ctx:
        q = torch.zeros(32, cfg.q_dim, device="cuda")
        with pytest.raises(GgrError) as e:
            ctx.attention_tokens_static(0, [4095] * 32, q)   # long context, few (sequence, kv head) groups: wants splits
        assert "static scratch too small" in str(e.value)
        # the same batch on a one-key context runs unsplit, needs no scratch and is accepted
        ctx.attention_tokens_static(0, [0] * 32, q)
        assert ctx.last_split_count == 1
        small = torch.zeros(2, cfg.q_dim, device="cuda")
        ctx.attention_tokens_static(0, [4095, 4095], small)  # a call within the limit still works afterwards
        torch.cuda.synchronize()
