"""CPU-side checks of the boundary: the shared library loads and exports every entry point that
include/uocr_rswa_b200.h declares (no compute call is made -- there is no GPU here)."""
import ctypes
import os

from paged_fixture import load_b200


def test_library_exports_every_declared_symbol():
    b = load_b200()
    if not os.path.exists(b.LIB_PATH):
        b.build()  # nvcc cross-compiles for sm_100a without a GPU
    names = b.declared_symbols()
    assert len(names) >= 15
    L = ctypes.CDLL(b.LIB_PATH)
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    # every declared function has a ctypes signature in the binding (kernel entry points) or is one
    # of the host-class wrappers of uocr_rswa_b200_host.h, and vice versa
    assert sorted(list(b._SIGS) + b.host_symbols()) == names
    b.lib()
    assert b.lib().uocr_b200_version().decode().endswith("sm_100a")
    assert b.lib().uocr_b200_status_string(4).decode() == "workspace too small"
