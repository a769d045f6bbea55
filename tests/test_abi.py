"""The C-ABI library builds, loads and exports every symbol include/ferrum_cuda.h declares. CPU only:
nothing here launches a kernel."""
import ctypes as C
import os
import re

import pytest

from ferrum_gpu_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_ffi.lib_path()):
        from ferrum_gpu_b200 import build
        build.build()
    return _ffi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ferrum_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fc_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in ferrum_cuda.h but not exported"
    assert set(names) == set(_ffi.EXPORTS), "the ctypes table and the header disagree"


def test_block_bytes_matches_the_gguf_sizes(lib):
    """ferrum_gguf/src/codec/quant.rs:L193-L207"""
    assert lib.fc_block_bytes(_ffi.FC_Q8_0, 64) == 68
    assert lib.fc_block_bytes(_ffi.FC_Q4_0, 64) == 36
    assert lib.fc_block_bytes(_ffi.FC_Q8_0, 33) == 0
    assert lib.fc_block_bytes(_ffi.FC_Q4_0, 31) == 0
    assert lib.fc_block_bytes(_ffi.FC_F32, 5) == 20


def test_plan_bytes_without_a_device(lib):
    """`plan` is pure arithmetic (models/llama/mod.rs:L108-L182): quantised plans are smaller, an
    invalid config plans nothing."""
    from ferrum_gpu_b200 import QKind, plan_bytes
    from ferrum_gpu_b200.hostmodel import config_c1, config_c3, config_c4
    c3 = config_c3()
    f32, q8, q4 = (plan_bytes(c3, k) for k in (None, QKind.Q8_0, QKind.Q4_0))
    assert f32 > q8 > q4 > 0
    mats = 12 * (768 * 1280 + 768 * 768 + 768 * 4096 + 2048 * 768) + 768 * 32000
    assert q4 >= mats * 18 // 32 and f32 >= mats * 4
    # C4: 64 streams of f32 KV dominate: 2 * 24 layers * 64 * 2048 * 128 * 4 bytes
    assert plan_bytes(config_c4(), QKind.Q8_0, 64) > 2 * 24 * 64 * 2048 * 128 * 4
    c3.kv_heads = 5
    assert plan_bytes(c3, QKind.Q4_0) == 0
    assert plan_bytes(config_c1(), QKind.Q8_0) > 0


def test_null_handles_are_refused_not_dereferenced(lib):
    assert lib.fc_device_close(None) == _ffi.FC_ERR_ARG
    assert lib.fc_qweight_destroy(None) == _ffi.FC_ERR_ARG
    assert lib.fc_model_destroy(None) == _ffi.FC_ERR_ARG
    assert lib.fc_device_sync(None) == _ffi.FC_ERR_ARG
    assert lib.fc_device_launch_count(None) == 0
    h = C.c_void_p()
    rc = lib.fc_device_open(-1, C.byref(h))
    assert rc != _ffi.FC_OK and not h.value
    assert lib.fc_last_error(None)  # a message, never NULL


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No CPU fallback: loading must raise when the built library is absent."""
    monkeypatch.setattr(_ffi, "_lib", None)
    monkeypatch.setattr(_ffi, "lib_path", lambda: str(tmp_path / "libferrum_cuda.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _ffi.load()
