"""The C-ABI library loads and exports every symbol that the headers under include/ declare. No GPU needed: nothing is
launched."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    inc = os.path.join(ROOT, "include")
    text = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(es_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_the_header():
    from self_trainable_or_free_attn_b200 import build
    lib = ctypes.CDLL(build.build())
    names = declared_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_covers_the_header():
    from self_trainable_or_free_attn_b200 import _native
    assert sorted(_native.SIGNATURES) == declared_symbols()
    lib = _native.load()
    assert lib.es_abi_version() == 1
    assert lib.es_reps_gram_splits(75600) == 32 and lib.es_reps_gram_splits(0) == 0


def test_argument_checks_come_before_any_launch():
    """Rejected calls return a negative code and a message; none of these reaches a kernel."""
    from self_trainable_or_free_attn_b200 import _native
    lib = _native.load()
    before = _native.launch_count()
    assert lib.es_block_means(None, None, None, None, 128, 1, None) < 0
    assert "null" in _native.last_error()
    assert lib.es_select_blocks(None, None, None, None, None, None, None, None, None, 4, None, 0, 1, 0, 128, 1, 1 << 30,
                                None) < 0
    assert lib.es_pack_plan(ctypes.c_void_p(16), ctypes.c_void_p(16), 1, 1, 1, 64, None) < 0     # 32 bits < 64 blocks
    assert "bits" in _native.last_error()
    assert _native.launch_count() == before


def test_missing_library_fails_loudly(monkeypatch):
    from self_trainable_or_free_attn_b200 import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", "/nonexistent/libechosparse_sm100.so")
    import pytest
    with pytest.raises(_native.NativeError, match="no CPU or Triton fallback"):
        _native.load()
