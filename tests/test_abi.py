"""CPU-side checks of the boundary: the library builds, loads and exports every declared symbol."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from streamdiffusionv2_b200 import build
    return build.build()


def test_header_symbols_are_exported(built_lib):
    header = open(os.path.join(ROOT, "include", "sdv2.h")).read()
    declared = set(re.findall(r"\b(sdv2_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(built_lib)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in sdv2.h but not exported"
    from streamdiffusionv2_b200 import _native
    assert set(_native.exported_symbols()) == declared


def test_version_and_messages(built_lib):
    from streamdiffusionv2_b200 import _native
    lib = _native.lib()
    assert lib.sdv2_abi_version() == 1
    assert lib.sdv2_strerror(0) == b"ok"
    assert b"aligned" in lib.sdv2_strerror(-3)
    assert lib.sdv2_attn_workspace_bytes(2, 3120, 12, 128) >= 256


def test_argument_validation_without_a_gpu(built_lib):
    """Validation happens before any CUDA call, so it can be exercised on a CPU-only box."""
    from streamdiffusionv2_b200 import _native as N
    lib = N.lib()
    v = N.View(0x1000, 128 * 4, 128, 128)
    bad = N.View(0x1008, 128 * 4, 128, 128)
    args = lambda q: [ctypes.byref(q)] * 4
    lens = N.i32_array([4])
    ws = 0x2000
    assert lib.sdv2_attn_kvcache(*args(v), 1, 4, 1, 64, 4, lens, 0.1, ws, 256, None) == -2     # head_dim
    assert lib.sdv2_attn_kvcache(*args(bad), 1, 4, 1, 128, 4, lens, 0.1, ws, 256, None) == -3  # alignment
    assert lib.sdv2_attn_kvcache(*args(v), 1, 4, 1, 128, 4, lens, 0.1, None, 0, None) == -6    # workspace
    assert lib.sdv2_attn_kvcache(*args(v), 1, 4, 1, 128, 3, lens, 0.1, ws, 256, None) == -1    # len > cache
    assert lib.sdv2_attn_kvcache(*args(v), 65, 4, 1, 128, 4, lens, 0.1, ws, 256, None) == -2   # rows


def test_no_fallback_when_library_missing(monkeypatch, tmp_path):
    from streamdiffusionv2_b200 import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _native.lib()
