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
    assert L.ggr_attn_abi_version() == 2
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


def test_header_is_valid_c99(tmp_path):
    """Rust FFI (and bindgen) consume the header as C: it must compile as strict C99 with no C++ around it."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use_header.c"
    src.write_text('#include "ggr_attn.h"\n'
                   "int use(void) { ggr_attn_config c; ggr_attn_config_init(&c); return (int)sizeof(c) + GGR_OK; }\n")
    proc = subprocess.run([cc, "-std=c99", "-pedantic", "-Wall", "-Werror", "-fsyntax-only",
                           "-I", os.path.join(ROOT, "include"), str(src)], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr


def test_rust_extern_block_names_every_function_with_the_headers_argument_count():
    """The Rust crate cannot be compiled here (no cargo); its extern block is at least held to the header."""
    text = open(os.path.join(ROOT, "include", "ggr_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    header = {}
    for name, args in re.findall(r"\b(ggr_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = " ".join(args.split())
        header[name] = 0 if args in ("", "void") else args.count(",") + 1
    rust = open(os.path.join(ROOT, "rust", "gguf-runner-cuda-sys", "src", "lib.rs")).read()
    block = rust[rust.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    decls = {}
    for name, args in re.findall(r"pub fn (ggr_[a-z0-9_]+)\(([^;]*?)\)\s*(?:->[^;]*)?;", block, flags=re.S):
        args = " ".join(args.split())
        decls[name] = 0 if not args else args.count(":")
    assert sorted(decls) == sorted(header)
    for name, n in header.items():
        assert decls[name] == n, name
    # the struct mirrors the C struct field for field
    c_fields = re.search(r"typedef struct ggr_attn_config \{(.*?)\} ggr_attn_config;", text, flags=re.S).group(1)
    c_names = [n.strip().split("[")[0].lstrip("*") for part in c_fields.split(";") if part.strip()
               for n in re.sub(r"^\s*(const\s+)?\w+\s*\*?", "", part.strip(), count=1).split(",")]
    r_fields = re.search(r"pub struct GgrAttnConfig \{(.*?)\n\}", rust, flags=re.S).group(1)
    r_names = re.findall(r"pub (\w+):", r_fields)
    assert r_names == c_names
