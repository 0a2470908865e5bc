"""The C-ABI library loads and exports every function include/fracssm.h declares (no GPU needed)."""

import ctypes
import os
import re

from frac_ssm_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header="fracssm.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fracssm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert "fracssm_frac_scan_fwd" in names and len(names) >= 14
    handle = ctypes.CDLL(_cabi.lib_path())
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"not exported: {missing}"


def test_selftest_library_exports_its_header_and_stays_out_of_the_product():
    names = _declared("fracssm_selftest.h")
    assert len(names) == 4
    product = ctypes.CDLL(_cabi.lib_path())
    selftest = ctypes.CDLL(os.path.join(os.path.dirname(_cabi.lib_path()), "libfracssm_selftest.so"))
    assert not [n for n in names if not hasattr(selftest, n)]
    assert not [n for n in names if hasattr(product, n)], "test-only entry points leaked into libfracssm.so"


def test_binding_covers_every_declared_symbol():
    assert sorted(_cabi._SIGNATURES) == _declared()


def test_abi_version_and_error_text():
    lib = _cabi.lib()
    assert lib.fracssm_abi_version() == _cabi.ABI_VERSION == 2
    # argument validation happens before any CUDA call, so this runs without a GPU
    rc = lib.fracssm_chunk_cumsum(None, 0, 0, 0, None, None, 1, 8, 0, 4, None)
    assert rc == 1
    assert b"chunk_cumsum" in lib.fracssm_last_error()
    rc = lib.fracssm_state_passing(None, 2, None, None, 0, None, 0, None, 0, 1, 1, 1, 1, None)
    assert rc == 1 and b"float32 or bfloat16" in lib.fracssm_last_error()
    assert lib.fracssm_frac_scan_workspace_bytes(2, 64, 8, 8, 16, 1) > 0
