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
