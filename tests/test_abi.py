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
    # the element-wise entry points
    a, odd = 0x1000, 0x1008
    assert lib.sdv2_gelu_tanh(None, a, 64, None) == -1                                          # null input
    assert lib.sdv2_gelu_tanh(a, a, 12, None) == -2                                             # not whole vectors
    assert lib.sdv2_gelu_tanh(odd, a, 64, None) == -3                                           # alignment
    assert lib.sdv2_layernorm_affine(a, a, a, a, 4, 5128, 1e-6, None) == -2                     # row too long
    assert lib.sdv2_layernorm_affine(a, a, None, a, 4, 1536, 1e-6, None) == -1                  # no bias
    assert lib.sdv2_layernorm_affine(a, odd, a, a, 4, 1536, 1e-6, None) == -3
    assert lib.sdv2_residual_layernorm(a, None, None, 0, a, 1, a, a, 0, a, 1, 1, 4, 1536, 1e-6, None) == -1   # no y
    assert lib.sdv2_residual_layernorm(a, a, a, 1000, a, 1, a, a, 0, a, 1, 1, 4, 1536, 1e-6, None) == -3      # gate rows overlap
    assert lib.sdv2_residual_layernorm(a, a, None, 0, a, 0, a, a, 1000, a, 1, 1, 4, 1536, 1e-6, None) == -3   # modulation rows overlap
    assert lib.sdv2_residual_layernorm(a, a, None, 0, a, 0, a, a, 9216, a, 1, 1, 4, 5128, 1e-6, None) == -2   # row too long


def test_no_fallback_when_library_missing(monkeypatch, tmp_path):
    from streamdiffusionv2_b200 import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _native.lib()


def test_tail_split_never_needs_more_than_the_fixed_scratch(built_lib):
    """The attention launcher and the allocation-free entry point share one split routine; for any
    SM count and problem it asks for at most 192 partial slots (what both scratch areas hold)."""
    from streamdiffusionv2_b200 import _native as N
    slots = N.lib().sdv2_attn_partial_slots
    # the production shape on a 148-SM part: 13 tile pairs x 12 heads x 2 rows = 312 = 2 x 148 + 16;
    # 148 // 16 = 9 key ranges per tail tile
    assert slots(2, 3120, 12, 32760, 148) == 16 * 9
    assert slots(2, 3120, 12, 15 * 128, 148) == 0          # key range too short to be worth a second launch
    assert slots(1, 256, 148, 32760, 148) == 0             # whole waves
    worst = 0
    for sms in (1, 7, 64, 108, 132, 148, 160, 192, 193, 256, 1024):
        for rows, q, heads in ((1, 256, 1), (2, 3120, 12), (4, 3120, 40), (16, 1560, 40), (64, 4680, 12), (3, 300, 5)):
            for seq in (128, 2047, 2048, 32760, 49920):
                n = slots(rows, q, heads, seq, sms)
                assert 0 <= n <= 192, (sms, rows, q, heads, seq, n)
                worst = max(worst, n)
    assert worst > 100      # the bound is actually approached, so the clamp matters
    assert slots(0, 1, 1, 1, 1) == 0 and slots(1, 1, 1, 1, 0) == 0
