"""The shared library must load without a GPU and export every function include/zant_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "zant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zant_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    assert len(names) >= 45
    for must in ("zant_b200_conv_f32", "zant_b200_qlinearconv", "zant_b200_plan_run", "zant_b200_gemm_f32"):
        assert must in names


def test_library_exports_every_declared_symbol(zb):
    lib = ctypes.CDLL(zb.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_version_and_status_names(zb):
    assert "sm_100a" in zb.version()
    L = zb.lib()
    assert L.zant_b200_status_name(ctypes.c_int32(-1)) == b"InvalidDimensions"
    assert L.zant_b200_status_name(ctypes.c_int32(-13)) == b"InvalidPadding"
    assert L.zant_b200_status_name(ctypes.c_int32(0)) == b"OK"


def test_product_never_touches_the_oracle():
    """No file of the package may include, import or load anything under oracle/."""
    pkg = os.path.join(ROOT, "z-ant_b200")
    for root, _d, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h", ".zig")):
                src = open(os.path.join(root, f), errors="ignore").read()
                assert "zant_oracle" not in src and "oracle/" not in src, os.path.join(root, f)
