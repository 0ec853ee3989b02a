"""The C-ABI library loads without a GPU and exports every function include/ggr_attn.h declares."""
import os
import re

import pytest

import gguf_runner_b200 as g
from gguf_runner_b200.binding import EXPORTED_SYMBOLS, GgrError, AttnConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ggr_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ggr_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_function_is_exported():
    L = g.lib()
    names = declared_functions()
    assert len(names) >= 30
    for name in names:
        assert hasattr(L, name), f"{name} is declared in ggr_attn.h but not exported"
    assert sorted(EXPORTED_SYMBOLS) == names


def test_abi_version_and_config_defaults():
    L = g.lib()
    assert L.ggr_attn_abi_version() == 1
    from gguf_runner_b200.binding import _Config
    import ctypes as C
    c = _Config()
    L.ggr_attn_config_init(C.byref(c))
    assert c.struct_size == C.sizeof(_Config)
    assert c.rope_theta == 500000.0 and c.rope_theta_swa == 10000.0 and c.swa_pattern == 6
    assert c.rope_scale_global == 1.0 and c.rope_scale_local == 1.0 and c.max_batch == 1


def test_create_without_a_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(GgrError):
        g.AttnContext(AttnConfig(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=8, seq_len=8))
