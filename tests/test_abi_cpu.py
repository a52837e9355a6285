"""CPU-side checks of the C ABI: the library loads without a GPU and exports
every function the header declares, and the ctypes table covers the header."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mytorch_b200.h")


def declared_in_header():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mt_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_header_symbols():
    from mytorch_b200 import _lib
    names = declared_in_header()
    assert len(names) > 50
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"


def test_ctypes_table_matches_header():
    from mytorch_b200 import _lib
    assert sorted(_lib.DECLARED) == declared_in_header()


def test_no_device_is_an_error_not_a_fallback():
    from mytorch_b200 import _lib
    import pytest
    if _lib.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(_lib.MTError):
        _lib.require_device()
    from mytorch_b200 import DeviceArray
    with pytest.raises(_lib.MTError):
        DeviceArray.empty((4,), "float32")


def test_argument_validation_happens_before_any_launch():
    from mytorch_b200 import _lib
    import pytest
    with pytest.raises(_lib.MTError) as e:
        _lib.layernorm_fwd(None, None, None, None, None, None, 4, 8, 1e-5, 0, None)
    assert "bad arguments" in str(e.value)
    with pytest.raises(_lib.MTError):
        _lib.gemm(1, 1, 1, None, None, 4, 4, 4, 2, 4, 4, 0, 0, 1, 1, 0, 1.0, 0, None)  # lda < K
