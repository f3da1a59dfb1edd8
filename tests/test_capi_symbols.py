"""The C-ABI shared library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes

import hipster_b200 as hb


def test_library_exports_every_declared_symbol():
    L = hb.lib()
    names = hb.declared_symbols()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_version_and_error_string_without_gpu():
    L = hb.lib()
    assert L.hp_version() >= 100
    assert isinstance(L.hp_last_error(), bytes)
    # argument validation happens before any CUDA call
    rc = L.hp_gemv_q4k_q8(ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), 16, 256, 1, 16, ctypes.c_void_p(0))
    assert rc == 1 and b"null" in L.hp_last_error()
    assert L.hp_xq8_q_bytes(3, 5120) == 5120 * 8 and L.hp_xq8_sc_bytes(9, 256) == 2 * 8 * 16 * 4
