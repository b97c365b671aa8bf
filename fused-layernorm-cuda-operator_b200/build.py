"""Build the native parts in-tree, for sm_100a only.

  libfln_b200.so                  CUDA kernels + C ABI (include/fln_b200.h); no torch
  fused_layernorm_cuda.<abi>.so   thin PyTorch extension over that C ABI: the module the
                                  reference builds with setup.py:5-12, same import name

Usage: python build.py [--force] [--verbose]
Both files land next to this script so that they travel with the source tree.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = HERE / "csrc"
INCLUDE = ROOT / "include"
OBJ = HERE / "build"
LIB = HERE / "libfln_b200.so"

CU_SOURCES = ["fln_pipeline_bwd_tail_bf16.cu", "fln_pipeline_bwd_tail_f16.cu", "fln_pipeline_bwd_tail_f32.cu", "fln_pipeline_bwd_odd.cu", "fln_pipeline_bwd.cu", "fln_pipeline_bwd_pair.cu", "fln_pipeline_bwd_wide.cu", "fln_pipeline_fwd.cu", "fln_pipeline_fwd_tail_bf16.cu", "fln_pipeline_fwd_tail_f16.cu", "fln_pipeline_fwd_tail_f32.cu", "fln_pipeline_fwd_fp8.cu", "fln_pipeline_fwd_drop.cu", "fln_forward.cu", "fln_backward.cu", "fln_fp8.cu", "fln_host.cu",
              "fln_pipeline.cu", "fln_static.cu", "fln_dropout.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)
    return r


def build_capi(force=False, verbose=False, ptxas_info=False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    sources = [s for s in CU_SOURCES if (CSRC / s).exists()]
    jobs = []
    for s in sources:
        src, obj = CSRC / s, OBJ / (s + ".o")
        if force or not _newer(obj, [src, *headers]):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for r in ex.map(lambda c: _run(c, verbose), jobs):
                if ptxas_info:
                    print(r.stderr)
    objs = [OBJ / (s + ".o") for s in sources]
    if force or jobs or not _newer(LIB, objs):
        _run([_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC"], verbose)
    return LIB


def shim_path() -> Path:
    return HERE / ("fused_layernorm_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_shim(force=False, verbose=False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    src = CSRC / "fln_torch_shim.cpp"
    out = shim_path()
    if not force and _newer(out, [src, LIB, *INCLUDE.glob("*.h")]):
        return out
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_home = Path(ce.CUDA_HOME or "/usr/local/cuda")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], str(INCLUDE), str(cuda_home / "include")]:
        inc += ["-isystem" if "torch" in p or "python" in p else "-I", p]
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared",
        "-DTORCH_EXTENSION_NAME=fused_layernorm_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
        "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi()),
        *inc, src, "-o", out,
        "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
        "-L", HERE, "-lfln_b200",
        "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + str(torch_lib),
    ]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False):
    lib = build_capi(force, verbose)
    shim = None
    if (CSRC / "fln_torch_shim.cpp").exists():
        shim = build_shim(force, verbose)
    return lib, shim


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers/spills per kernel")
    a = ap.parse_args()
    if a.ptxas_info:
        build_capi(True, a.verbose, True)
    else:
        print(build_all(a.force, a.verbose))
