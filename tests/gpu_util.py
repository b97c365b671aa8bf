"""Helpers for the GPU parity tests: seeded inputs generated on the CPU (so the oracle and the
kernels see identical bits), guarded device buffers, and calls through the C ABI."""
from __future__ import annotations

import torch

from fused_layernorm import _capi as capi
from oracle import oracle as O

GUARD = 64  # elements of sentinel after every output buffer
KINDS = {"layernorm": capi.LAYERNORM, "rmsnorm": capi.RMSNORM}
ACTS = {"none": capi.ACT_NONE, "gelu_tanh": capi.ACT_GELU_TANH, "gelu_erf": capi.ACT_GELU_ERF}


def make_inputs(seed, rows, cols, dtype, x_scale=1.0, x_shift=0.0, residual=False, outliers=False,
                affine=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * x_scale + x_shift
    if outliers:
        x = torch.where(torch.rand(rows, cols, generator=g) < 0.001, x * 50.0, x)
    gamma = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(dtype) if affine else None
    beta = (0.1 * torch.randn(cols, generator=g)).to(dtype) if affine else None
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    res = (0.5 * torch.randn(rows, cols, generator=g)).to(dtype) if residual else None
    return x.to(dtype), gamma, beta, dy, res


def dev(t):
    return None if t is None else t.cuda()


class Guarded:
    """Device buffer of `shape` followed by GUARD sentinel elements; .check() asserts that the
    sentinel is untouched (the bounds check that stands in for a memory sanitizer)."""

    def __init__(self, shape, dtype, fill=None):
        n = 1
        for s in shape:
            n *= s
        self.n = n
        self.dtype = dtype
        self.buf = torch.empty(n + GUARD, dtype=dtype, device="cuda")
        self.sentinel = 77 if dtype == torch.uint8 else 12345.0
        self.buf.fill_(self.sentinel)
        self.t = self.buf[:n].view(*shape)
        if fill is not None:
            self.t.fill_(fill)

    def check(self):
        tail = self.buf[self.n:]
        assert bool((tail == self.sentinel).all()), "kernel wrote past the end of its output"
        return self.t


def run_forward(x, gamma, beta, res=None, kind="layernorm", eps=1e-5, act="none", out_dtype=None,
                want_stats=True):
    rows, cols = x.shape
    xd, gd, bd, rd = dev(x), dev(gamma), dev(beta), dev(res)
    y = Guarded((rows, cols), out_dtype or x.dtype)
    s = Guarded((rows, cols), x.dtype) if res is not None else None
    mean = Guarded((rows,), torch.float32) if (want_stats and kind == "layernorm") else None
    rstd = Guarded((rows,), torch.float32) if want_stats else None
    capi.norm_forward(KINDS[kind], xd, rd, gd, bd, y.t, s.t if s else None, mean.t if mean else None,
                      rstd.t if rstd else None, eps, ACTS[act])
    torch.cuda.synchronize()
    return {"y": y.check().cpu(), "sum": s.check().cpu() if s else None,
            "mean": mean.check().cpu() if mean else None, "rstd": rstd.check().cpu() if rstd else None}


def run_backward(dy, x, mean, rstd, gamma, kind="layernorm", dres_in=None, want=(True, True, True),
                 with_f32=True):
    rows, cols = x.shape
    dt = x.dtype
    nr = 2 if kind == "layernorm" else 1
    dx = Guarded((rows, cols), dt) if want[0] else None
    dg = Guarded((cols,), dt) if want[1] else None
    db = Guarded((cols,), dt) if (want[2] and kind == "layernorm") else None
    f32 = Guarded((nr * cols,), torch.float32) if with_f32 else None
    nbytes = capi.backward_workspace_bytes(rows, cols, dt)
    ws = Guarded((max(nbytes // 4, 1),), torch.float32)
    capi.norm_backward(KINDS[kind], dev(dy), dev(x), dev(mean), dev(rstd), dev(gamma), dev(dres_in),
                       dx.t if dx else None, dg.t if dg else None, db.t if db else None,
                       f32.t if f32 else None, ws.t if nbytes else None)
    torch.cuda.synchronize()
    ws.check()
    return {"dx": dx.check().cpu() if dx else None, "dgamma": dg.check().cpu() if dg else None,
            "dbeta": db.check().cpu() if db else None, "dgb_f32": f32.check().cpu() if f32 else None}


def assert_out_close(a, b, dtype, tol=1e-5):
    """fp32: 1e-5 abs/rel.  bf16/fp16: at most one unit in the last place (oracle.mismatch_16)."""
    if dtype == torch.float32:
        torch.testing.assert_close(a.float(), b.float(), rtol=tol, atol=tol)
    else:
        bad = O.mismatch_16(a, b)
        assert int(bad.sum()) == 0, f"{int(bad.sum())} elements off by more than 1 ulp"


def assert_param_grads_close(got_f32, want64, abs64, rows):
    """dgamma/dbeta are sums of `rows` signed terms that may cancel; judge the fp32 result
    against the float64 oracle relative to the sum of |terms| (fp32 accumulation error grows
    like eps * sum|terms|), with the usual 1e-5 on top."""
    tol = 1e-5 * want64.abs() + 1e-5 + 4e-7 * abs64
    err = (got_f32.double() - want64).abs()
    assert bool((err <= tol).all()), f"max excess {(err - tol).max().item():.3e}"
