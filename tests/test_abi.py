"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_eagle.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_symbols()
    assert "b200_qmm" in names and "b200_qmm_fused" in names


def test_library_exports_every_declared_symbol(be):
    lib = be._lib.lib()
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/b200_eagle.h but not exported"


def test_version_and_error_codes_without_gpu(be):
    lib = be._lib.lib()
    assert lib.b200_version() >= 1
    # argument validation happens before any CUDA call, so it can be exercised on CPU
    rc = lib.b200_qmm(None, None, None, None, None, None, 8, 64, 100, 64, 0, None, 0, None)
    assert rc == -1
    rc = lib.b200_qmm(None, None, None, None, None, None, 8, 64, 128, 32, 0, None, 0, None)
    assert rc == -3
    buf = (ctypes.c_char * 64)()
    base = ctypes.addressof(buf)
    base += (-base) % 16
    rc = lib.b200_qmm(base + 2, base, base, base, None, base, 8, 64, 128, 64, 0, None, 0, None)
    assert rc == -2


def test_workspace_query(be):
    assert be.qmm_kernel.workspace_bytes(16, 152064, 3584) == 0      # wide layer: no split-K
    assert be.qmm_kernel.workspace_bytes(16, 3584, 18944) > 4096     # narrow, deep layer: split-K


def test_exchange_buffer_size_query(be):
    lib = be._lib.lib()
    # header, two buffers of partial products (fp32), two gather areas (fp16), two sets of 8 push slots (fp32), 32 rows each
    for hidden in (896, 3584, 8192):
        assert lib.b200_forward_tp_buffer_bytes(hidden) == 4096 + 32 * hidden * (2 * 4 + 2 * 2 + 2 * 8 * 4)
    assert lib.b200_forward_tp_buffer_bytes(100) == 0 and lib.b200_forward_tp_buffer_bytes(0) == 0


def test_missing_library_fails_loudly(be, monkeypatch):
    import pytest
    monkeypatch.setattr(be._lib, "_lib", None)
    monkeypatch.setattr(be._lib, "LIB_PATH", "/nonexistent/libb200eagle.so")
    with pytest.raises(be._lib.B200Error):
        be._lib.lib()


def test_forward_descriptor_validation_without_gpu(be):
    lib = be._lib.lib()
    d = be._lib.ForwardDesc()
    d.M, d.rows_out = 16, 16
    d.hidden, d.intermediate, d.n_heads, d.n_kv_heads, d.head_dim = 3584, 18944, 28, 4, 128
    d.vocab, d.n_layers, d.cache_rows, d.write_off, d.tail = 152064, 28, 1024, 0, 16
    assert lib.b200_forward_workspace_bytes(ctypes.byref(d)) > 4352
    assert lib.b200_forward(ctypes.byref(d), None) == -1          # null pointers: refused before any CUDA call
    d.hidden = 3500                                               # not a multiple of 128
    assert lib.b200_forward_workspace_bytes(ctypes.byref(d)) == 0
    d.hidden, d.head_dim = 3584, 96
    assert lib.b200_forward(ctypes.byref(d), None) == -1
    assert ctypes.sizeof(be._lib.ForwardDesc) == 64 + 20 * 8 + 8 + 16 + 16 + 64 + 8 + 8  # layout of b200_forward_desc in the header
