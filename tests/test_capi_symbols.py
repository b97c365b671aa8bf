"""The C-ABI library loads and exports every symbol include/fln_b200.h declares.
No kernel is launched here; only host-side entry points are called."""
import ctypes as C
import re
from pathlib import Path

import torch

from fused_layernorm import _capi as capi

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "fln_b200.h").read_text()


def declared_symbols():
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(fln_[a-z0-9_]+)\s*\(", code)))


def test_every_declared_symbol_is_exported():
    lib = C.CDLL(str(capi.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_table_matches_header():
    assert sorted(capi.SYMBOLS) == declared_symbols()


def test_host_only_entry_points():
    lib = capi.lib()
    assert lib.fln_version().decode() == "1.0.0"
    assert lib.fln_cuda_runtime_version() >= 12000
    assert lib.fln_status_string(0).decode() == "ok"
    assert "workspace" in lib.fln_status_string(4).decode()
    # same closed form as the reference's get_memory_usage (csrc/layernorm_cuda.cpp:144-164)
    b, h = 32, 4096
    for mixed, e in ((0, 4), (1, 2)):
        want = 2 * b * h * e + 2 * b * 4 + b * h * e + 2 * h * e + b * 32 * 4
        assert lib.fln_get_memory_usage(b, h, mixed) == want
    buf = C.create_string_buffer(1024)
    n = lib.fln_get_performance_hints(4, 1000, buf, 1024)
    text = buf.value.decode()
    assert n == len(text) and "not divisible by 32" in text and "Small batch size" in text
    small = C.create_string_buffer(8)
    assert lib.fln_get_performance_hints(4, 1000, small, 8) == n and len(small.value) == 7


def test_launch_planner_without_a_device():
    info = capi.describe_launch(False, 16384, 8192, torch.bfloat16)
    assert info["generic"] == 0 and info["vec_elems"] == 8 and info["threads_per_row"] * info["vecs_per_thread"] == 1024
    assert info["pipelined"] == 1 and info["stages"] >= 2 and info["vector_bytes"] == 16
    # 5120 = 5 * 1024: backward gives every thread 5 vectors of 4 columns, forward 5 of 4 elements
    b5 = capi.describe_launch(True, 16384, 5120, torch.bfloat16)
    assert b5["pipelined"] == 1 and b5["vecs_per_thread"] == 5 and b5["vector_bytes"] == 8 and b5["threads_per_row"] == 256
    f3 = capi.describe_launch(False, 16384, 768, torch.bfloat16)
    assert f3["pipelined"] == 1 and f3["vecs_per_thread"] == 3 and f3["threads_per_row"] == 32
    small = capi.describe_launch(False, 32, 4096, torch.bfloat16)
    assert small["pipelined"] == 0
    odd = capi.describe_launch(False, 17, 1023, torch.bfloat16)
    assert odd["vec_elems"] == 1 and odd["generic"] == 0
    huge = capi.describe_launch(False, 1, 100000, torch.float32)
    assert huge["generic"] == 1
    bwd = capi.describe_launch(True, 64, 2048, torch.float32)
    assert bwd["vec_elems"] * bwd["vecs_per_thread"] <= 32


def test_pipeline_planner_invariants_over_a_grid_of_shapes():
    """Every plan the pipeline planner accepts (forward with one or two staged tensors, backward
    with two or three, 16-bit and fp32, row lengths that are and are not powers of two) describes
    a launch that exists; checked on the host, no GPU needed."""
    assert capi.lib().fln_planner_selftest() == 0


def test_argument_errors_are_status_codes_not_crashes():
    lib = capi.lib()
    null = None
    # bad dtype / shape / enum are rejected before anything touches a device
    assert lib.fln_layernorm_forward(null, null, null, null, null, null, 4, 8, 7, 1e-5, null) == 1
    assert lib.fln_layernorm_forward(null, null, null, null, null, null, 4, 0, 0, 1e-5, null) == 2
    assert lib.fln_layernorm_forward(null, null, null, null, null, null, 4, 8, 0, 1e-5, null) == 3
    assert lib.fln_norm_forward(5, null, null, null, null, null, null, null, null, 4, 8, 0, 0, 1e-5, 0, null) == 8
    assert lib.fln_layernorm_gelu_forward(null, null, null, null, 4, 8, 0, 1e-5, 0, null) == 8
    assert lib.fln_norm_backward(0, null, null, null, null, null, null, null, null, null, null, null, 0, 4, 8, 9,
                                 null) == 1
    assert lib.fln_backward_workspace_bytes(0, 8, 0) == 0
