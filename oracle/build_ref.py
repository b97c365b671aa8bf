"""Compiles the reference's own shipped extension (csrc/bindings.cpp +
csrc/layernorm_cuda_kernel.cu, the two files its setup.py:7-10 builds) for sm_100, from the
sources where they lie, into oracle/_ref/.  Nothing is copied or modified; the only change
is the module name (-DTORCH_EXTENSION_NAME=ref_g2_layernorm_cuda) so that it cannot be
confused with this repository's fused_layernorm_cuda.

CHECKER ONLY: the built module is used to produce tests/golden/ref_g2_b200.npz on a B200 and
for cross-checks in GPU tests; the product never loads it.  It does not use the reference's
setup.py (its own build system), only nvcc and g++ directly.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "ref_g2_layernorm_cuda"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FLN_REFERENCE_DIR"), required="FLN_REFERENCE_DIR" not in os.environ,
                    help="checkout of the reference (or set FLN_REFERENCE_DIR)")
    a = ap.parse_args()
    ref = Path(a.reference)
    srcs = [ref / "csrc" / "bindings.cpp", ref / "csrc" / "layernorm_cuda_kernel.cu"]
    for s in srcs:
        if not s.exists():
            sys.exit(f"{s} not found")
    import torch
    from torch.utils import cpp_extension as ce

    OUT.mkdir(exist_ok=True)
    so = OUT / (NAME + sysconfig.get_config_var("EXT_SUFFIX"))
    if so.exists() and all(so.stat().st_mtime >= s.stat().st_mtime for s in srcs):
        print(so)
        return
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_home = Path(ce.CUDA_HOME or "/usr/local/cuda")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], str(cuda_home / "include")]:
        inc += ["-isystem", p]
    defs = [f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi())]
    o_cpp, o_cu = OUT / "bindings.o", OUT / "kernel.o"
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", *defs, *inc, "-c", str(srcs[0]), "-o", str(o_cpp)], check=True)
    subprocess.run([str(cuda_home / "bin" / "nvcc"), "-O3", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100",
                    "-Xcompiler", "-fPIC", *defs, *inc, "-c", str(srcs[1]), "-o", str(o_cu)], check=True)
    subprocess.run(["g++", "-shared", str(o_cpp), str(o_cu), "-o", str(so), "-L", str(torch_lib), "-lc10", "-lc10_cuda",
                    "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L", str(cuda_home / "lib64"),
                    "-lcudart", "-Wl,-rpath," + str(torch_lib)], check=True)
    o_cpp.unlink()
    o_cu.unlink()
    print(so)


if __name__ == "__main__":
    main()
