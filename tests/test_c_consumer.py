"""include/fln_b200.h is a C header: a C11 translation unit compiles against it with warnings as
errors, links libfln_b200.so and calls the host-side entry points.  No GPU needed."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "fused-layernorm-cuda-operator_b200"


def test_c11_consumer_compiles_links_and_runs(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    assert (PKG / "libfln_b200.so").exists(), "build the library first (python build.py)"
    exe = tmp_path / "consumer"
    cmd = [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "c_consumer" / "consumer.c"), "-L", str(PKG), "-lfln_b200",
           "-Wl,-rpath," + str(PKG), "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "c consumer ok" in r.stdout


def test_header_also_compiles_as_cxx(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    src = tmp_path / "tu.cpp"
    src.write_text('#include "fln_b200.h"\nint main() { return fln_version() == nullptr; }\n')
    r = subprocess.run([gxx, "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", str(ROOT / "include"), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
