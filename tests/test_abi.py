"""The C ABI and the Python mirror without a GPU: symbols, status codes, argument checks."""
import ctypes
import os
import re

import pytest
import torch

import tinyfa_b200
from tinyfa_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tinyfa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tfa_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 7
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared


def test_head_dim_table():
    for d in (32, 64, 96, 128, 192, 256):
        assert tinyfa_b200.is_head_dim_compiled(d)
    for d in (0, 16, 48, 80, 160, 512):
        assert not tinyfa_b200.is_head_dim_compiled(d)


def test_status_codes_for_bad_arguments():
    """Argument validation happens before any device work, so it can be exercised on a CPU-only host."""
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 15) & ~15
    f = lib.tfa_b200_fwd
    assert f(p, p, p, p, 9, 1, 16, 16, 1, 1, 64, 0, None) == 1  # dtype
    assert "dtype" in _lib.last_error()
    assert f(p, p, p, p, 1, 1, 16, 16, 1, 1, 80, 0, None) == 2  # head dim
    assert "unsupported headDim: 80" in _lib.last_error()
    assert f(p, p, p, p, 1, 1, 16, 16, 6, 4, 64, 0, None) == 3  # Hq % Hkv
    assert f(p, p, p, p, 1, -1, 16, 16, 4, 4, 64, 0, None) == 3  # negative size
    assert f(None, p, p, p, 1, 1, 16, 16, 4, 4, 64, 0, None) == 3  # null
    assert f(p + 4, p, p, p, 1, 1, 16, 16, 4, 4, 64, 0, None) == 3  # alignment
    assert f(p, p, p, p, 1, 70000, 16, 16, 4, 4, 64, 0, None) == 6  # grid limit
    # nothing to do: success without touching a device
    assert f(p, p, p, p, 1, 0, 16, 16, 4, 4, 64, 0, None) == 0
    assert f(p, p, p, p, 1, 2, 16, 0, 4, 4, 64, 0, None) == 0
    v = lib.tfa_b200_fwd_varlen
    assert v(p, p, p, p, None, None, 1, 2, 16, 16, 32, 32, 4, 4, 64, 0, None) == 3  # null cu_seqlens
    assert v(p, p, p, p, p, p, 1, 0, 16, 16, 0, 0, 4, 4, 64, 0, None) == 0
    assert lib.tfa_b200_set_option(b"no_such_option", 1) == 3
    assert lib.tfa_b200_set_option(b"pack_gqa", -1) == 0
    # every option the header documents is known to the library; -1 / 1 are their documented defaults
    for name, default in ((b"split_kv", -1), (b"narrow_mma", 1), (b"solo64", 1), (b"pair_cta", -1), (b"fp32_t8", 1), (b"work_order", -1)):
        assert lib.tfa_b200_set_option(name, default) == 0, name


def test_python_mirror_rejects_like_the_reference_binding():
    """Every violated precondition is a RuntimeError (reference csrc/binding/flash_attn_binding.cu:84-104,125-146)."""
    q = torch.zeros(1, 4, 2, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        tinyfa_b200.flash_attn_forward(q, q, q)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        tinyfa_b200.flash_attn_varlen_forward(q[0], q[0], q[0], torch.zeros(2, dtype=torch.int32),
                                              torch.zeros(2, dtype=torch.int32), 4, 4)


def test_module_name_of_the_reference_package():
    import tiny_flash_attn

    assert tiny_flash_attn.flash_attn_forward is tinyfa_b200.flash_attn_forward
    assert tiny_flash_attn.flash_attn_varlen_forward is tinyfa_b200.flash_attn_varlen_forward
    import inspect

    sig = inspect.signature(tiny_flash_attn.flash_attn_forward)
    assert list(sig.parameters) == ["Q", "K", "V", "is_causal"] and sig.parameters["is_causal"].default is False
    sig = inspect.signature(tiny_flash_attn.flash_attn_varlen_forward)
    assert list(sig.parameters) == ["Q", "K", "V", "cu_seqlens_q", "cu_seqlens_kv", "max_seqlen_q", "max_seqlen_kv",
                                    "is_causal"]


def test_product_never_touches_the_oracle():
    """The shipped packages must not import, load or mention the checker."""
    for pkg in ("tinyfa_b200", "tiny_flash_attn"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, pkg)):
            if os.sep + "build" in dirpath:
                continue
            for fn in files:
                if fn.endswith((".py", ".cu", ".cuh", ".h")):
                    text = open(os.path.join(dirpath, fn)).read()
                    assert "oracle" not in text.lower(), os.path.join(dirpath, fn)
