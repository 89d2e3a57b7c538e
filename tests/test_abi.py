"""CPU tests of the drop-in boundary: the C-ABI library loads without a GPU and exports every symbol that
include/*.h declares; the Python binding refuses to work without the library (no CPU fallback)."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names.update(re.findall(r"\b(simp_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    import simplang_b200 as sg
    lib = ctypes.CDLL(sg.LIB_PATH)
    syms = declared_symbols()
    assert len(syms) >= 30
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_binding_covers_the_header():
    import simplang_b200 as sg
    sg.lib()
    bound = set(sg._SIGNATURES) | {"simp_gpu_last_error", "simp_gpu_stream"}
    undeclared = bound - set(declared_symbols())
    assert not undeclared, f"bound in Python but not declared in the header: {undeclared}"


def test_no_silent_fallback_without_the_library(monkeypatch, tmp_path):
    import simplang_b200 as sg
    monkeypatch.setattr(sg, "_LIB", None)
    monkeypatch.setattr(sg, "LIB_PATH", str(tmp_path / "missing.so"))
    try:
        sg.lib()
    except ImportError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("expected ImportError")


def test_product_does_not_import_the_oracle():
    for path in glob.glob(os.path.join(ROOT, "simplang_b200", "**", "*"), recursive=True):
        if path.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
            text = open(path, errors="ignore").read()
            assert "import oracle" not in text and "simp_oracle" not in text and "oracle/" not in text, path


def test_cpp_host_builds_and_reports_a_missing_library():
    import subprocess
    from simplang_b200 import build as b
    exe = b.build_host()
    r = subprocess.run([exe, "/nonexistent/libsimp_gpu.so"], capture_output=True, text=True)
    assert r.returncode == 1 and "Failed to load library" in r.stderr


def test_host_matmul_quant_rejects_out_of_range_shapes_before_touching_a_device():
    """The host-pointer W4 entry and its memref shim know the real array sizes: a wrong offset / rows / cols must
    come back as SIMP_ERR_SHAPE (-2) without any device work (none is possible here: no GPU)."""
    import numpy as np
    import simplang_b200 as sg
    L = sg.lib()
    rows, cols, gs = 8, 256, 64
    qw = np.zeros(rows * cols // 2, np.uint8)
    sc = np.ones(rows * cols // gs, np.float32)
    x = np.zeros(cols, np.float32)
    out = np.zeros(rows, np.float32)
    p = lambda a: a.ctypes.data

    def call(rows_, cols_, offset, mode, n_groups=sc.size, qw_bytes=qw.nbytes):
        return L.simp_host_matmul_quant(p(qw), qw_bytes, p(sc), None, n_groups, p(x), p(out), rows_, cols_, gs, offset, mode)

    assert call(rows + 1, cols, 0, 1) == -2 and b"qweights" in L.simp_gpu_last_error()
    assert call(rows, cols, 64, 1) == -2                      # offset pushes the last row past the end
    assert call(rows, cols, 0, 1, n_groups=sc.size - 1) == -2 and b"group" in L.simp_gpu_last_error()
    assert call(rows, cols, 0, 2) == -1
    assert call(rows, cols, -1, 1) == -1
    # the shim takes rows / cols from the call and the lengths from the memref descriptors
    i64 = ctypes.c_int64
    def memref1(a):
        return [ctypes.c_void_p(p(a)), ctypes.c_void_p(p(a)), i64(0), i64(a.size), i64(1)]
    zr = np.zeros_like(sc)
    L.simp_rt_matmul_quant.argtypes = None
    rc = L.simp_rt_matmul_quant(*memref1(qw), *memref1(sc), *memref1(zr), *memref1(x), *memref1(out),
                                i64(rows), i64(cols + 64), i64(gs), i64(0))
    assert rc == -2 and b"exceed" in L.simp_gpu_last_error()
    rc = L.simp_rt_matmul_quant(*memref1(qw), *memref1(sc), *memref1(zr), *memref1(x), *memref1(out),
                                i64(rows + 1), i64(cols), i64(gs), i64(0))
    assert rc == -2
