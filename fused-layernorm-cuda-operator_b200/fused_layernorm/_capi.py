"""ctypes binding of the C ABI in include/fln_b200.h (libfln_b200.so).

This is the binding a maintainer of the reference would add in place of its pybind launchers
(csrc/bindings.cpp:19-39, csrc/layernorm_cuda.cpp:49-141 of the reference): tensors are passed
as raw device pointers plus sizes, the stream as an integer handle, and every call returns a
status code that is turned into a RuntimeError here.  There is no CPU path: if the library is
missing, importing the symbols raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_PKG_DIR = Path(__file__).resolve().parents[1]
LIB_PATH = _PKG_DIR / "libfln_b200.so"

F32, BF16, F16, FP8_E4M3 = 0, 1, 2, 3
LAYERNORM, RMSNORM = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

# every symbol include/fln_b200.h declares
SYMBOLS = [
    "fln_status_string", "fln_version", "fln_cuda_runtime_version",
    "fln_layernorm_forward", "fln_layernorm_gelu_forward", "fln_norm_forward", "fln_norm_forward_fp8",
    "fln_backward_workspace_bytes", "fln_layernorm_backward", "fln_norm_backward", "fln_cast_from_f32",
    "fln_graph_begin", "fln_graph_stream", "fln_graph_end", "fln_graph_launch", "fln_graph_destroy",
    "fln_get_memory_usage", "fln_get_performance_hints", "fln_describe_launch", "fln_set_plan_override",
    "fln_set_path_override", "fln_device_status", "fln_layernorm_backward_static", "fln_set_sm_reserve",
    "fln_norm_forward_fp8_delayed", "fln_norm_forward_fp8_rowwise", "fln_norm_forward_mxfp8",
    "fln_planner_selftest", "fln_sum_rows_f32", "fln_set_stage_override", "fln_set_wait_limit_ns",
    "fln_set_test_fault", "fln_set_static_scratch_limit", "fln_norm_backward_partial", "fln_dropout_add_norm_forward", "fln_dropout_backward", "fln_norm_forward_nvfp4",
]
STATIC_SCRATCH_BYTES = 24 << 20  # FLN_STATIC_SCRATCH_BYTES


class LaunchInfo(C.Structure):
    _fields_ = [("generic", C.c_int), ("vec_elems", C.c_int), ("vecs_per_thread", C.c_int),
                ("threads_per_row", C.c_int), ("threads_per_cta", C.c_int), ("rows_per_cta", C.c_int),
                ("grid", C.c_int64), ("sm_count", C.c_int), ("pipelined", C.c_int), ("stages", C.c_int),
                ("vector_bytes", C.c_int)]


_lib = None


def lib() -> C.CDLL:
    """Load libfln_b200.so (once).  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found. Build it with `python {_PKG_DIR / 'build.py'}`; "
            "this package has no CPU or pure-PyTorch fallback.")
    L = C.CDLL(str(LIB_PATH))
    vp, i64, i32, f32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t
    L.fln_status_string.restype = C.c_char_p
    L.fln_status_string.argtypes = [i32]
    L.fln_version.restype = C.c_char_p
    L.fln_cuda_runtime_version.restype = i32
    L.fln_layernorm_forward.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_layernorm_gelu_forward.argtypes = [vp, vp, vp, vp, i64, i64, i32, f32, i32, vp]
    L.fln_norm_forward.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, f32, i32, vp]
    L.fln_norm_forward_fp8.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_norm_forward_fp8_delayed.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_norm_forward_fp8_rowwise.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_norm_forward_mxfp8.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_norm_forward_nvfp4.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, vp]
    L.fln_backward_workspace_bytes.restype = sz
    L.fln_backward_workspace_bytes.argtypes = [i64, i64, i32]
    L.fln_layernorm_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, vp]
    L.fln_norm_backward.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, vp]
    L.fln_norm_backward_partial.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, vp, C.POINTER(i64)]
    u64 = C.c_ulonglong
    L.fln_dropout_add_norm_forward.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, f32, u64, u64, vp]
    L.fln_dropout_backward.argtypes = [vp, vp, vp, i64, i64, i32, f32, u64, u64, vp]
    L.fln_cast_from_f32.argtypes = [vp, vp, i64, i32, vp]
    L.fln_sum_rows_f32.argtypes = [vp, i64, i64, vp, vp, i32, vp]
    L.fln_set_stage_override.restype = None
    L.fln_set_stage_override.argtypes = [i32]
    L.fln_set_wait_limit_ns.argtypes = [C.c_ulonglong]
    L.fln_set_test_fault.argtypes = [i32]
    L.fln_set_static_scratch_limit.restype = None
    L.fln_set_static_scratch_limit.argtypes = [sz]
    L.fln_graph_begin.argtypes = [C.POINTER(vp)]
    L.fln_graph_stream.restype = vp
    L.fln_graph_stream.argtypes = [vp]
    L.fln_graph_end.argtypes = [vp]
    L.fln_graph_launch.argtypes = [vp, vp]
    L.fln_graph_destroy.argtypes = [vp]
    L.fln_get_memory_usage.restype = i64
    L.fln_get_memory_usage.argtypes = [i32, i32, i32]
    L.fln_get_performance_hints.argtypes = [i32, i32, C.c_char_p, sz]
    L.fln_describe_launch.argtypes = [i32, i64, i64, i32, i32, C.POINTER(LaunchInfo)]
    L.fln_set_plan_override.argtypes = [i32, i32]
    L.fln_set_plan_override.restype = None
    L.fln_set_path_override.argtypes = [i32]
    L.fln_set_path_override.restype = None
    L.fln_device_status.restype = i32
    L.fln_set_sm_reserve.argtypes = [i32]
    L.fln_set_sm_reserve.restype = None
    L.fln_layernorm_backward_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, vp]
    _lib = L
    return L


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what}: {lib().fln_status_string(status).decode()} (status {status})")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_handle(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPES[t.dtype]
    except KeyError:
        raise NotImplementedError(f'"layernorm" not implemented for {t.dtype}') from None


# ----------------------------------------------------------------------------------------
# thin wrappers: device tensors in, device tensors out; the caller allocates
# ----------------------------------------------------------------------------------------
def norm_forward(kind, x, residual, gamma, beta, y, sum_out, mean, rstd, eps, act=ACT_NONE, stream=None):
    rows, cols = x.shape
    out_dt = DTYPES[y.dtype]
    check(lib().fln_norm_forward(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(y), ptr(sum_out),
                                 ptr(mean), ptr(rstd), rows, cols, dtype_code(x), out_dt, eps, act,
                                 stream_handle(stream)), "fln_norm_forward")


def layernorm_forward(x, gamma, beta, y, mean, rstd, eps, stream=None):
    rows, cols = x.shape
    check(lib().fln_layernorm_forward(ptr(x), ptr(gamma), ptr(beta), ptr(y), ptr(mean), ptr(rstd), rows,
                                      cols, dtype_code(x), eps, stream_handle(stream)),
          "fln_layernorm_forward")


def layernorm_gelu_forward(x, gamma, beta, y, eps, approximate=ACT_GELU_TANH, stream=None):
    rows, cols = x.shape
    check(lib().fln_layernorm_gelu_forward(ptr(x), ptr(gamma), ptr(beta), ptr(y), rows, cols, dtype_code(x),
                                           eps, approximate, stream_handle(stream)),
          "fln_layernorm_gelu_forward")


def norm_forward_fp8(kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax, scale, eps, stream=None):
    rows, cols = x.shape
    check(lib().fln_norm_forward_fp8(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(q),
                                     ptr(sum_out), ptr(mean), ptr(rstd), ptr(amax), ptr(scale), rows, cols,
                                     dtype_code(x), eps, stream_handle(stream)), "fln_norm_forward_fp8")


def norm_forward_fp8_delayed(kind, x, residual, gamma, beta, q, sum_out, mean, rstd, scale_in, amax_out, eps,
                             stream=None):
    """One launch: q = sat_e4m3(y * scale_in[0]); amax_out (optional) receives max|y| of this call."""
    rows, cols = x.shape
    check(lib().fln_norm_forward_fp8_delayed(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(q),
                                             ptr(sum_out), ptr(mean), ptr(rstd), ptr(scale_in), ptr(amax_out),
                                             rows, cols, dtype_code(x), eps, stream_handle(stream)),
          "fln_norm_forward_fp8_delayed")


def norm_forward_fp8_rowwise(kind, x, residual, gamma, beta, q, sum_out, mean, rstd, row_scale, amax_out, eps,
                             stream=None):
    """One launch: row_scale[r] = 448 / max|y[r]|, q[r] = sat_e4m3(y[r] * row_scale[r])."""
    rows, cols = x.shape
    check(lib().fln_norm_forward_fp8_rowwise(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(q),
                                             ptr(sum_out), ptr(mean), ptr(rstd), ptr(row_scale), ptr(amax_out),
                                             rows, cols, dtype_code(x), eps, stream_handle(stream)),
          "fln_norm_forward_fp8_rowwise")


def norm_forward_mxfp8(kind, x, residual, gamma, beta, q, block_scale, sum_out, mean, rstd, amax_out, eps,
                       stream=None):
    """One launch: MXFP8 output, one E8M0 scale byte per 32 consecutive elements of a row
    (block_scale: uint8 [rows, cols // 32]); q = sat_e4m3(y / 2^(byte - 127))."""
    rows, cols = x.shape
    check(lib().fln_norm_forward_mxfp8(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(q), ptr(block_scale),
                                       ptr(sum_out), ptr(mean), ptr(rstd), ptr(amax_out), rows, cols, dtype_code(x),
                                       eps, stream_handle(stream)), "fln_norm_forward_mxfp8")


def dropout_add_norm_forward(kind, x, residual, gamma, beta, y, sum_out, mean, rstd, keep_bits, eps, p, seed, offset,
                             stream=None):
    """y = norm(dropout(x, p) + residual); keep_bits (uint8 [rows * cols / 8], optional) receives the mask."""
    rows, cols = x.shape
    check(lib().fln_dropout_add_norm_forward(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(y), ptr(sum_out),
                                             ptr(mean), ptr(rstd), ptr(keep_bits), rows, cols, dtype_code(x), eps, p,
                                             seed, offset, stream_handle(stream)), "fln_dropout_add_norm_forward")


def dropout_backward(d_sum, keep_bits, d_x, p, seed, offset, stream=None):
    rows, cols = d_sum.shape
    check(lib().fln_dropout_backward(ptr(d_sum), ptr(keep_bits), ptr(d_x), rows, cols, dtype_code(d_sum), p, seed,
                                     offset, stream_handle(stream)), "fln_dropout_backward")


def norm_forward_nvfp4(kind, x, residual, gamma, beta, q, block_scale, sum_out, mean, rstd, tensor_scale, amax_out, eps,
                       stream=None):
    """One launch: NVFP4-style output.  q: uint8 [rows, cols // 2] (two e2m1 per byte), block_scale:
    uint8 [rows, cols // 16] (e4m3), tensor_scale: one fp32 on the device."""
    rows, cols = x.shape
    check(lib().fln_norm_forward_nvfp4(kind, ptr(x), ptr(residual), ptr(gamma), ptr(beta), ptr(q), ptr(block_scale),
                                       ptr(sum_out), ptr(mean), ptr(rstd), ptr(tensor_scale), ptr(amax_out), rows, cols,
                                       dtype_code(x), eps, stream_handle(stream)), "fln_norm_forward_nvfp4")


def backward_workspace_bytes(rows, cols, dtype) -> int:
    return int(lib().fln_backward_workspace_bytes(rows, cols, DTYPES[dtype]))


def norm_backward(kind, dy, x, mean, rstd, gamma, dres_in, dx, dgamma, dbeta, dgb_f32, workspace, stream=None):
    rows, cols = x.shape
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(lib().fln_norm_backward(kind, ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma), ptr(dres_in),
                                  ptr(dx), ptr(dgamma), ptr(dbeta), ptr(dgb_f32), ptr(workspace), ws_bytes,
                                  rows, cols, dtype_code(x), stream_handle(stream)), "fln_norm_backward")


def norm_backward_partial(kind, dy, x, mean, rstd, gamma, dres_in, dx, workspace, stream=None):
    """Stage 1 only: dx and the unreduced partial sums.  Returns them as a view [P, NR * cols]
    of `workspace` (fp32); add its rows with sum_rows_f32, on any stream."""
    rows, cols = x.shape
    n = C.c_int64(0)
    ws_bytes = workspace.numel() * workspace.element_size()
    check(lib().fln_norm_backward_partial(kind, ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma), ptr(dres_in), ptr(dx),
                                          ptr(workspace), ws_bytes, rows, cols, dtype_code(x), stream_handle(stream),
                                          C.byref(n)), "fln_norm_backward_partial")
    nr = 2 if kind == LAYERNORM else 1
    return workspace.view(torch.float32).reshape(-1)[: n.value * nr * cols].view(n.value, nr * cols)


def layernorm_backward(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, workspace, stream=None):
    rows, cols = x.shape
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(lib().fln_layernorm_backward(ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma), ptr(dx),
                                       ptr(dgamma), ptr(dbeta), ptr(workspace), ws_bytes, rows, cols,
                                       dtype_code(x), stream_handle(stream)), "fln_layernorm_backward")


def layernorm_backward_static(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, stream=None):
    """LayerNorm backward for hosts that may not allocate device memory: no workspace argument,
    the partial sums live in an array built into the library (at most STATIC_SCRATCH_BYTES;
    larger problems raise).  Make the first call on a device outside stream capture, and do
    not let two calls overlap on the GPU: they share that array."""
    rows, cols = x.shape
    check(lib().fln_layernorm_backward_static(ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma), ptr(dx),
                                              ptr(dgamma), ptr(dbeta), rows, cols, dtype_code(x),
                                              stream_handle(stream)), "fln_layernorm_backward_static")


def cast_from_f32(src, dst, stream=None):
    check(lib().fln_cast_from_f32(ptr(src), ptr(dst), src.numel(), DTYPES[dst.dtype], stream_handle(stream)),
          "fln_cast_from_f32")


def sum_rows_f32(rows_in, out_f32=None, out_cast=None, stream=None):
    """Fixed-order column sum of an fp32 matrix [n, ncols] into out_f32 and / or out_cast."""
    n, ncols = rows_in.shape
    dt = DTYPES[out_cast.dtype] if out_cast is not None else F32
    check(lib().fln_sum_rows_f32(ptr(rows_in), n, ncols, ptr(out_f32), ptr(out_cast), dt, stream_handle(stream)),
          "fln_sum_rows_f32")


def describe_launch(backward, rows, cols, dtype, aligned16=True) -> dict:
    info = LaunchInfo()
    check(lib().fln_describe_launch(int(backward), rows, cols, DTYPES[dtype], int(aligned16), C.byref(info)),
          "fln_describe_launch")
    return {f: getattr(info, f) for f, _ in LaunchInfo._fields_}


class Graph:
    """Record a sequence of C-ABI launches once, replay it with one CUDA-graph launch.

        g = Graph()
        with g.record() as s:          # s: a torch.cuda.ExternalStream to launch on
            layernorm_forward(x, w, b, y, None, None, 1e-5, stream=s)
        g.launch()                     # on the current stream
    """

    def __init__(self):
        self._h = C.c_void_p()
        self._recorded = False

    def record(self):
        return _GraphRecorder(self)

    def launch(self, stream=None):
        if not self._recorded:
            raise RuntimeError("graph has not been recorded")
        check(lib().fln_graph_launch(self._h, stream_handle(stream)), "fln_graph_launch")

    def close(self):
        if self._h:
            lib().fln_graph_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _GraphRecorder:
    def __init__(self, g):
        self.g = g

    def __enter__(self):
        check(lib().fln_graph_begin(C.byref(self.g._h)), "fln_graph_begin")
        return torch.cuda.ExternalStream(lib().fln_graph_stream(self.g._h))

    def __exit__(self, et, ev, tb):
        if et is not None:
            self.g.close()
            return False
        check(lib().fln_graph_end(self.g._h), "fln_graph_end")
        self.g._recorded = True
        return False
