"""The C-ABI library builds, loads and exports every symbol that the headers under include/ declare
(no kernel is launched here)."""
import ctypes
import re

from conftest import ROOT


def _declared():
    text = "".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pamk_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from pam_b200 import _lib, build
    path = build.build()
    handle = ctypes.CDLL(str(path))
    names = _declared()
    assert len(names) >= 15
    for name in names:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_lib.exported_names()), "ctypes signatures out of sync with the header"
    assert handle.pamk_abi_version() >= 1
    _lib.lib().pamk_status_string(-3).decode().startswith("matrix operand")


def test_argument_checks_need_no_gpu():
    # validation happens before any CUDA call, so these statuses are observable on a CPU box
    from pam_b200 import _lib
    h = _lib.lib()
    assert h.pamk_pam_fwd(None, 0, 0.0, None, 0, 0.0, None, 8, 0, 1.0, None) == -1        # null operands
    assert h.pamk_pam_fwd(None, 4, 1.0, None, 4, 2.0, None, -1, 0, 1.0, None) == -1       # negative size
    assert h.pamk_pam_fwd(None, 4, 1.0, None, 4, 2.0, None, 0, 0, 1.0, None) == 0         # empty is fine
    assert h.pamk_matmul(7, None, None, None, 1, 1, 1, 1, 0, 1, 1, 0, 1, 1, 1.0, 1, None, 0, None) == -1
    one = ctypes.c_float(1.0)
    ptr = ctypes.addressof(one)
    # a matrix whose two strides are both != 1 cannot be addressed
    assert h.pamk_matmul(0, ptr, ptr, ptr, 1, 4, 4, 4, 0, 8, 2, 0, 4, 1, 1.0, 1, None, 0, None) == -3
    assert h.pamk_matmul(0, ptr, ptr, ptr, 1, 2**31, 4, 4, 0, 4, 1, 0, 4, 1, 1.0, 1, None, 0, None) == -2
    assert h.pamk_matmul(0, ptr, ptr, ptr, 1, 4, 4, 64, 0, 64, 1, 0, 4, 1, 1.0, 4, None, 0, None) == -4
    assert h.pamk_matmul_workspace_bytes(2, 3, 5, 4) == 2 * 3 * 5 * 4 * 4


def test_nvtx_wrapper_marks_only_entry_points_that_launch():
    """With tracing on, entry points that take a stream are wrapped in an NVTX range; helpers that only
    compute sizes or plans are passed through untouched."""
    from pam_b200 import _lib
    plain = _lib.lib()
    _lib.set_nvtx(True)
    try:
        traced = _lib.lib()
        assert traced is not plain
        assert traced.pamk_matmul_auto_split(1, 64, 64, 64) == plain.pamk_matmul_auto_split(1, 64, 64, 64)
        assert traced.pamk_softmax_max_len is not None and not hasattr(traced.pamk_softmax_max_len, "__wrapped_name__")
        assert getattr(traced.pamk_matmul, "__name__", "") == "wrapped"
        assert getattr(traced.pamk_matmul_workspace_bytes, "__name__", "") != "wrapped"
    finally:
        _lib.set_nvtx(False)
    assert _lib.lib() is plain
