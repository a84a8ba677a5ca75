"""The C-ABI library loads without a GPU and exports every symbol that include/qtip_b200.h declares."""
import os
import re

import pytest

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


def test_size_queries_and_host_heuristics(pkg):
    """Workspace / exchange sizes and the K-split heuristics of the host mirror: pure host logic, no device."""
    import ctypes as C
    lib = pkg.Library()
    ex = lib.cdll.qtip_tp_exchange_bytes
    one = ex(57344, 1, 1)
    assert one == 256 + 2 * ((57344 * 4 + 255) // 256 * 256)          # control block + two slots
    assert ex(57344, 16, 4) == 256 + 2 * 57344 * 16 * 4 * 4
    assert ex(0, 1, 1) == 0
    ldlq = lib.cdll.qtip_ldlq_workspace_bytes(28672, 12288)
    assert ldlq >= 28672 * 12288 * 4 + 768 * 16 * 4096 * 4                # prod + back-pointers of every sequence
    assert lib.cdll.qtip_quantize_linear_workspace_bytes(12288, 28672) > ldlq
    assert C.sizeof(pkg.QtipTpExchange) == 8 * 8 + 8 + 4 + 4 and C.sizeof(pkg.QtipMatrix) == 4 * 8 + 4 + 4
    lin = pkg.linear
    assert lin.tc_splits(12288) == 3 and lin.tc_splits(57344) == 4 and lin.tc_splits(128) == 4
    assert lin.fp8_splits(12288, 1024, 64) == 37 and lin.fp8_splits(12288, 1024, 2048) == 4
    assert lin.fp8_splits(1536, 128, 19) == 6
    # exchange argument checks that need no device: bad rank count, bad slot
    bad = pkg.QtipTpExchange()
    bad.ranks, bad.rank, bad.bytes = 9, 0, 4096
    assert lib.cdll.qtip_gathered_products(C.byref(bad), 0, C.byref(C.c_void_p())) == -1


@pytest.mark.parametrize("unit,defines,includes", [
    ("shim_signatures_quantizer.cpp", ["-DQTIP_CUDA"], ["src", "third_party"]),
    ("shim_signatures_runtime.cpp", ["-DGLM53_CUDA=1"], ["runtime/cuda", "runtime/include", "glm53/include", "third_party"]),
])
def test_reference_side_shims_match_the_reference_headers(unit, defines, includes):
    """The binding headers a maintainer of the reference would add (include/shims/) are compiled against the
    reference's own headers; static_asserts compare every forwarding function's type with the declaration it replaces."""
    import shutil
    import subprocess
    from conftest import REFERENCE_ROOT, ROOT
    if not os.path.isdir(os.path.join(REFERENCE_ROOT, "src")):
        pytest.skip("reference tree not present")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"))), "include")
    cmd = [cxx, "-std=c++20", "-fsyntax-only", *defines, "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc,
           *["-I" + os.path.join(REFERENCE_ROOT, d) for d in includes], os.path.join(ROOT, "tests", unit)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
