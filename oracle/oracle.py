"""ctypes front end of the CPU checker (oracle/fln_oracle.c) plus the torch-CPU composition
the reference's own tests treat as ground truth.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / --impl reference legs of bench.py.  The product never imports this module.

All functions take and return CPU torch tensors.  bf16 / fp16 tensors are handed to C as raw
16-bit words; the C side does its own conversions, so nothing here depends on torch's
rounding except the fixtures it is pinned against.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
_LIB_PATH = HERE / "_build" / "libfln_oracle.so"

DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
KIND = {"layernorm": 0, "rmsnorm": 1}
ACT = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2, "tanh": 1, "erf": 2}


def build(force: bool = False) -> Path:
    """Compile oracle/fln_oracle.c with gcc (via the Makefile) if the library is missing."""
    src = HERE / "fln_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE)] + (["-B"] if force else []), check=True,
                       capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB_PATH))
        vp, i64, i32, f32p, dbl, f64p = C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_double, C.c_void_p
        L.oracle_norm_forward.argtypes = [i32, vp, vp, vp, vp, vp, f32p, vp, f32p, f32p, i64, i64, i32, i32, dbl, i32]
        L.oracle_norm_forward.restype = None
        L.oracle_norm_backward.argtypes = [i32, vp, vp, f32p, f32p, vp, vp, vp, f32p, vp, vp, f64p, f64p, f64p, i64, i64, i32]
        L.oracle_norm_backward.restype = None
        L.oracle_quant_fp8.argtypes = [f32p, i64, f32p, f32p, vp]
        L.oracle_quant_fp8.restype = None
        L.ref_g2_layernorm_f32.argtypes = [f32p, f32p, f32p, f32p, i64, i32, C.c_float, i32]
        L.ref_g2_layernorm_f32.restype = None
        L.oracle_convert_from_f32.argtypes = [f32p, vp, i64, i32]
        L.oracle_convert_to_f32.argtypes = [vp, f32p, i64, i32]
        L.oracle_e4m3_encode.argtypes = [f32p, vp, i64]
        L.oracle_quant_nvfp4.argtypes = [f32p, i64, i64, C.c_float, vp, vp, vp]
        L.oracle_e2m1_decode.argtypes = [C.c_uint8]
        L.oracle_e2m1_decode.restype = C.c_float
        L.oracle_e4m3_decode.argtypes = [C.c_uint8]
        L.oracle_e4m3_decode.restype = C.c_float
        L.oracle_philox4x32_10.argtypes = [vp, vp, vp]
        L.oracle_dropout_keep_bits.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, i64, vp]
        L.oracle_dropout_apply.argtypes = [vp, vp, vp, i64, i32, C.c_float]
        _lib = L
    return _lib


def _ptr(t):
    if t is None:
        return None
    assert t.device.type == "cpu" and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def _c(t):
    return None if t is None else t.detach().contiguous()


def norm_forward(x, gamma=None, beta=None, residual=None, kind="layernorm", eps=1e-5, act="none",
                 out_dtype=None):
    """Double-accumulator restatement of the forward.  Returns a dict with y (out dtype),
    y32 (fp32 value before the last rounding), sum (x + residual in the I/O type, or None),
    mean and rstd (fp32 [rows]; mean is None for rmsnorm)."""
    x = _c(x)
    rows, cols = x.shape
    io = x.dtype
    out_dtype = out_dtype or io
    gamma, beta, residual = _c(gamma), _c(beta), _c(residual)
    for p in (gamma, beta, residual):
        assert p is None or p.dtype == io
    y = torch.empty(rows, cols, dtype=out_dtype)
    y32 = torch.empty(rows, cols, dtype=torch.float32)
    s = torch.empty_like(x) if residual is not None else None
    mean = torch.empty(rows, dtype=torch.float32) if kind == "layernorm" else None
    rstd = torch.empty(rows, dtype=torch.float32)
    lib().oracle_norm_forward(KIND[kind], _ptr(x), _ptr(residual), _ptr(gamma), _ptr(beta), _ptr(y),
                              _ptr(y32), _ptr(s), _ptr(mean), _ptr(rstd), rows, cols, DT[io],
                              DT[out_dtype], float(eps), ACT[act])
    return {"y": y, "y32": y32, "sum": s, "mean": mean, "rstd": rstd}


def norm_backward(dy, x, mean, rstd, gamma=None, dres_in=None, kind="layernorm"):
    """Double-accumulator backward from saved fp32 mean / rstd.  Returns dx (I/O dtype), dx32,
    dgamma / dbeta (I/O dtype), dgamma64 / dbeta64 (float64) and abs64 ([2, cols] float64: the
    sums of |terms|, the scale for judging sums that cancel)."""
    dy, x, gamma, dres_in = _c(dy), _c(x), _c(gamma), _c(dres_in)
    rows, cols = x.shape
    dt = x.dtype
    dx = torch.empty_like(x)
    dx32 = torch.empty(rows, cols, dtype=torch.float32)
    dgamma = torch.empty(cols, dtype=dt)
    dbeta = torch.empty(cols, dtype=dt) if kind == "layernorm" else None
    dg64 = torch.empty(cols, dtype=torch.float64)
    db64 = torch.empty(cols, dtype=torch.float64)
    abs64 = torch.empty(2, cols, dtype=torch.float64)
    mean = _c(mean) if mean is not None else None
    lib().oracle_norm_backward(KIND[kind], _ptr(dy), _ptr(x), _ptr(mean), _ptr(_c(rstd)), _ptr(gamma),
                               _ptr(dres_in), _ptr(dx), _ptr(dx32), _ptr(dgamma), _ptr(dbeta),
                               _ptr(dg64), _ptr(db64), _ptr(abs64), rows, cols, DT[dt])
    return {"dx": dx, "dx32": dx32, "dgamma": dgamma, "dbeta": dbeta, "dgamma64": dg64,
            "dbeta64": db64 if kind == "layernorm" else None, "abs64": abs64}


def quant_fp8(y32):
    """amax, scale = 448/amax (fp32), q = saturating e4m3 codes (uint8) of y32 * scale."""
    y32 = _c(y32).float()
    q = torch.empty(y32.shape, dtype=torch.uint8)
    amax = torch.zeros(1, dtype=torch.float32)
    scale = torch.zeros(1, dtype=torch.float32)
    lib().oracle_quant_fp8(_ptr(y32), y32.numel(), _ptr(amax), _ptr(scale), _ptr(q))
    return q, amax, scale


def quant_fp8_delayed(y32, scale):
    """Quantization with a scale fixed beforehand (delayed scaling): q = saturating e4m3 of
    y32 * scale, and amax = max |y32| of this tensor for the next step.  The torch composition
    is (y32 * scale).clamp(-448, 448).to(float8_e4m3fn); y32.abs().max()."""
    y32 = _c(y32).float()
    q = e4m3_encode(y32 * torch.as_tensor(scale, dtype=torch.float32).reshape(()))
    return q, y32.abs().max().reshape(1)


def quant_fp8_rowwise(y32):
    """One scale per row: scale[r] = 448 / max |y32[r]| in fp32 (1 for an all-zero row),
    q[r] = saturating e4m3 of y32[r] * scale[r]."""
    y32 = _c(y32).float()
    rmax = y32.abs().amax(dim=-1)
    scale = torch.where(rmax > 0, torch.tensor(448.0) / rmax, torch.ones_like(rmax))
    q = e4m3_encode(y32 * scale[:, None])
    return q, scale, rmax.max().reshape(1) if rmax.numel() else torch.zeros(1)


def quant_mxfp8(y32, e8m0=None):
    """OCP microscaling MXFP8: blocks of 32 consecutive elements of a row share the scale
    2^(floor(log2(block max)) - 8), stored as the E8M0 byte floor(log2(max)) - 8 + 127 (0 for a
    block whose maximum is below 2^-119, zero included); elements are saturating e4m3 codes of
    y / scale.  Returns (codes uint8 [rows, cols], scale bytes uint8 [rows, cols // 32]).  With
    `e8m0` given, those scale bytes are used instead of being derived."""
    y32 = _c(y32).float()
    rows, cols = y32.shape
    blocks = y32.reshape(rows, cols // 32, 32)
    if e8m0 is None:
        amax = blocks.abs().amax(dim=-1)
        expf = (amax.view(torch.int32) >> 23) & 0xFF          # biased exponent = floor(log2) + 127
        e8m0 = torch.clamp(expf - 8, min=0).to(torch.uint8)
    inv = torch.pow(2.0, 127.0 - e8m0.to(torch.float64)).to(torch.float32)  # exact powers of two
    q = e4m3_encode((blocks * inv[..., None]).reshape(rows, cols))
    return q, e8m0


def ref_g2_layernorm(x, gamma, beta, eps=1e-5, gelu=False):
    """Literal fp32 restatement of the reference's shipped kernel, summation order included."""
    x = _c(x).float()
    rows, cols = x.shape
    y = torch.empty_like(x)
    lib().ref_g2_layernorm_f32(_ptr(x), _ptr(_c(gamma)), _ptr(_c(beta)), _ptr(y), rows, cols,
                               C.c_float(eps), int(bool(gelu)))
    return y


def convert_from_f32(src, dtype):
    src = _c(src).float()
    out = torch.empty(src.shape, dtype=dtype)
    lib().oracle_convert_from_f32(_ptr(src), _ptr(out), src.numel(), DT[dtype])
    return out


def e4m3_encode(src):
    src = _c(src).float()
    out = torch.empty(src.shape, dtype=torch.uint8)
    lib().oracle_e4m3_encode(_ptr(src), _ptr(out), src.numel())
    return out


# --------------------------------------------------------------------------------------
# torch-CPU composition: what the reference's tests compare against
# (tests/test_layernorm.py:47-178 -> nn.LayerNorm / F.layer_norm and autograd), extended
# with the unfused compositions for the variants the reference does not have.
# --------------------------------------------------------------------------------------
def torch_forward(x, gamma=None, beta=None, residual=None, kind="layernorm", eps=1e-5, act="none",
                  out_dtype=None):
    io = x.dtype
    out_dtype = out_dtype or io
    s = x if residual is None else (x + residual)  # rounded to the I/O type, like unfused torch
    sf = s.float()
    g = None if gamma is None else gamma.float()
    b = None if beta is None else beta.float()
    if kind == "layernorm":
        y32, mean, rstd = torch.native_layer_norm(sf, (sf.shape[-1],), g, b, eps)
        mean, rstd = mean.reshape(-1), rstd.reshape(-1)
    else:
        y32 = F.rms_norm(sf, (sf.shape[-1],), g, eps)
        mean, rstd = None, torch.rsqrt(sf.pow(2).mean(-1) + eps)
    if act in ("gelu_tanh", "tanh"):
        y32 = F.gelu(y32, approximate="tanh")
    elif act in ("gelu_erf", "erf"):
        y32 = F.gelu(y32)
    return {"y": y32.to(out_dtype), "y32": y32, "sum": None if residual is None else s, "mean": mean,
            "rstd": rstd}


def torch_backward(dy, x, gamma=None, beta=None, kind="layernorm", eps=1e-5):
    """Autograd through the float64 composition on the (already rounded) inputs."""
    xd = x.double().requires_grad_(True)
    gd = None if gamma is None else gamma.double().requires_grad_(True)
    bd = None if beta is None else beta.double().requires_grad_(True)
    if kind == "layernorm":
        y = F.layer_norm(xd, (x.shape[-1],), gd, bd, eps)
    else:
        y = F.rms_norm(xd, (x.shape[-1],), gd, eps)
    y.backward(dy.double())
    return {"dx": xd.grad, "dgamma": None if gd is None else gd.grad,
            "dbeta": None if bd is None else bd.grad}


def torch_quant_fp8(y32):
    amax = y32.abs().max()
    scale = (448.0 / amax).float() if amax > 0 else torch.tensor(1.0)
    q = (y32 * scale).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), amax.reshape(1), scale.reshape(1)


# --------------------------------------------------------------------------------------
# tolerance helpers shared by the tests
# --------------------------------------------------------------------------------------
def ulp_distance_16(a, b):
    """|difference| in units of the last place between two bf16 (or two fp16) tensors,
    via their monotone integer encodings."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()


def fp8_code_distance(a_u8, b_u8):
    def key(t):
        i = t.to(torch.int32)
        return torch.where(i >= 128, -(i & 0x7F), i)
    return (key(a_u8) - key(b_u8)).abs()


def mismatch_16(a, b, abs_floor=1e-5):
    """Elements of two bf16 (or fp16) tensors that differ by more than one unit in the last
    place AND by more than abs_floor in value.  The floor is the fp32 tolerance of the
    computation underneath: where the result is a near-zero difference of fp32 quantities
    (e.g. GELU of a large negative input) a bound in ulps of the tiny result is meaningless."""
    ulp = ulp_distance_16(a, b)
    return (ulp > 1) & ((a.float() - b.float()).abs() > abs_floor)


def philox4x32_10(ctr, key):
    """One block of Philox4x32-10: ctr (4 uint32), key (2 uint32) -> 4 uint32."""
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().oracle_philox4x32_10(c.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    return out


def dropout_threshold(p: float):
    """(threshold, scale) the library derives from p: drop iff 16 random bits < threshold."""
    thr = min(int(p * 65536.0 + 0.5), 65535)
    return thr, float(np.float32(65536.0 / (65536.0 - thr)))


def dropout_keep_bits(seed: int, offset: int, p: float, n_elements: int):
    """uint8 [n_elements / 8]: bit j of byte g = element 8 g + j is kept."""
    assert n_elements % 8 == 0
    bits = torch.zeros(n_elements // 8, dtype=torch.uint8)
    thr, _ = dropout_threshold(p)
    lib().oracle_dropout_keep_bits(seed, offset, thr, n_elements // 8, _ptr(bits))
    return bits


def dropout_apply(x, bits, p: float):
    """round(x / (1 - p')) where kept, 0 elsewhere, in the dtype of x (forward and backward alike)."""
    x = _c(x)
    out = torch.empty_like(x)
    _, scale = dropout_threshold(p)
    lib().oracle_dropout_apply(_ptr(x), _ptr(bits), _ptr(out), x.numel(), DT[x.dtype], scale)
    return out


E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def quant_nvfp4(y32, tensor_scale: float, block_scales=None):
    """NVFP4-style quantization of y32 [rows, cols]: (q uint8 [rows, cols // 2] with element 2 i in
    the low nibble, block scales uint8 [rows, cols // 16] in e4m3).  With block_scales given,
    those are used instead of being derived."""
    y32 = _c(y32).float()
    rows, cols = y32.shape
    q = torch.empty(rows, cols // 2, dtype=torch.uint8)
    bs = torch.empty(rows, cols // 16, dtype=torch.uint8)
    lib().oracle_quant_nvfp4(_ptr(y32), rows, cols, float(tensor_scale), _ptr(_c(block_scales)), _ptr(q), _ptr(bs))
    return q, bs


def dequant_nvfp4(q, block_scales, tensor_scale: float):
    """fp32 [rows, cols] from the packed e2m1 codes, the e4m3 block scales and the tensor scale."""
    rows, half = q.shape
    lut = torch.tensor(E2M1_VALUES + [-v for v in E2M1_VALUES], dtype=torch.float32)
    lo, hi = lut[(q & 15).long()], lut[(q >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(rows, half * 2)
    e4 = torch.tensor([lib().oracle_e4m3_decode(c) for c in range(256)], dtype=torch.float32)
    f = e4[block_scales.long()].repeat_interleave(16, dim=1)
    return vals * f / tensor_scale
