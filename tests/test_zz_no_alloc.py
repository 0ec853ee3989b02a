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
from gguf_runner_b200.binding import AttnConfig, GgrError, KV_BF16, KV_Q8_ROW

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_format,n_heads,n_kv_heads", [(KV_BF16, 16, 2), (KV_Q8_ROW, 4, 2)])
def test_static_scratch_entry_matches_regular_entry(kv_format, n_heads, n_kv_heads):
    import torch
    B, T = 3, 3000
    cfg = AttnConfig(n_layers=2, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=128, seq_len=T, max_batch=B,
                     rope_theta=1e6, kv_format=kv_format)
    rng = np.random.default_rng(17)
    with g.AttnContext(cfg) as ctx:
        lens = [T - 1, 2000, 700]
        for b, n in enumerate(lens):
            q = rng.standard_normal((n, cfg.q_dim)).astype(np.float32)
            k = rng.standard_normal((n, cfg.kv_dim)).astype(np.float32)
            v = rng.standard_normal((n, cfg.kv_dim)).astype(np.float32)
            ctx.prefill(1, 0, q, k, v, seq=b)
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
        assert ctx.launch_count > launches


def test_static_scratch_entry_rejects_oversized_calls():
    import torch
    # 2 * B * n_heads * (head_dim + 2) floats must fit the built-in 8 MiB array
    cfg = AttnConfig(n_layers=1, n_heads=128, n_kv_heads=8, head_dim=256, seq_len=64, max_batch=128,
                     kv_format=KV_BF16)
    with g.AttnContext(cfg) as ctx:
        q = torch.zeros(128, cfg.q_dim, device="cuda")
        with pytest.raises(GgrError) as e:
            ctx.attention_tokens_static(0, [0] * 128, q)
        assert "static scratch too small" in str(e.value)
        small = torch.zeros(2, cfg.q_dim, device="cuda")
        ctx.attention_tokens_static(0, [0, 0], small)  # a call within the limit still works afterwards
        torch.cuda.synchronize()
