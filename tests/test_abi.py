"""The C-ABI library loads without a GPU and exports every symbol that include/qtip_b200.h declares."""
import os
import re

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qtip_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qtip_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    lib = pkg.Library()
    names = declared_functions()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib.cdll, name), "libqtip_b200.so does not export %s" % name


def test_binding_covers_header(pkg):
    assert set(declared_functions()) <= set(pkg.exported_names())


def test_abi_version_and_error_string(pkg):
    lib = pkg.Library()
    assert lib.cdll.qtip_abi_version() == 1
    assert isinstance(lib.last_error(), str)


def test_argument_checks_need_no_device(pkg):
    """Geometry and null-pointer violations are rejected before any CUDA call."""
    lib = pkg.Library()
    import ctypes as C
    assert lib.cdll.qtip_quantize_tiles(None, 4, None, None, None, None, 0, None) == -1
    assert lib.cdll.qtip_swizzle_for_kernel(C.c_void_p(16), 48, 64, C.c_void_p(16), None) == -2
    assert "multiples of 32" in lib.last_error()
    assert lib.cdll.qtip_ldlq(C.c_void_p(16), C.c_void_p(16), 100, 64, 0, 64, C.c_void_p(16), C.c_void_p(16),
                              C.c_void_p(16), C.c_void_p(16), 1 << 20, None) == -2
    assert lib.cdll.qtip_quantize_workspace_bytes(8) >= 8 * 16 * 4096 * 4
