"""torch.library registrations for the operators the extension defines (fused_layernorm::*).

The C++ side (csrc/fln_torch_shim.cpp) declares the schemas and the CUDA implementations; this
module adds what tracing needs: a fake (meta) implementation per operator, so torch.compile /
make_fx can propagate shapes without running a kernel, and autograd formulas for the forward
operators, expressed with the backward operators.  The reference wires autograd by hand in
FusedLayerNormFunction (fused_layernorm/layernorm.py:31-109 of the reference) and registers no
operators at all; its pybind functions are opaque to torch.compile.
"""
from __future__ import annotations

import torch

import fused_layernorm_cuda  # noqa: F401  (loads the TORCH_LIBRARY block; raises if not built)

ops = torch.ops.fused_layernorm
LAYERNORM, RMSNORM = 0, 1


def _stat(x):
    return x.new_empty((x.shape[0],), dtype=torch.float32)


def _none_if_empty(t):
    return None if t is None or t.numel() == 0 else t


# ------------------------------------------------------------------------------------ fakes
@torch.library.register_fake("fused_layernorm::layernorm")
def _(input, gamma, beta, epsilon):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake("fused_layernorm::layernorm_gelu")
def _(input, gamma, beta, epsilon, approximate):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake("fused_layernorm::layernorm_fwd")
def _(input, gamma, beta, epsilon):
    return torch.empty_like(input, memory_format=torch.contiguous_format), _stat(input), _stat(input)


@torch.library.register_fake("fused_layernorm::rmsnorm_fwd")
def _(input, gamma, epsilon):
    return torch.empty_like(input, memory_format=torch.contiguous_format), _stat(input)


@torch.library.register_fake("fused_layernorm::add_layernorm_fwd")
def _(input, residual, gamma, beta, epsilon):
    e = lambda: torch.empty_like(input, memory_format=torch.contiguous_format)
    return e(), e(), _stat(input), _stat(input)


@torch.library.register_fake("fused_layernorm::add_rmsnorm_fwd")
def _(input, residual, gamma, epsilon):
    e = lambda: torch.empty_like(input, memory_format=torch.contiguous_format)
    return e(), e(), _stat(input)


@torch.library.register_fake("fused_layernorm::norm_fp8")
def _(kind, input, residual, gamma, beta, epsilon):
    q = input.new_empty(input.shape, dtype=torch.float8_e4m3fn)
    s = torch.empty_like(input, memory_format=torch.contiguous_format) if residual is not None else input.new_empty((0,))
    mean = _stat(input) if kind == LAYERNORM else input.new_empty((0,), dtype=torch.float32)
    return q, s, input.new_empty((1,), dtype=torch.float32), mean, _stat(input)


@torch.library.register_fake("fused_layernorm::norm_fp8_scaled")
def _(kind, input, residual, gamma, beta, scale_in, epsilon):
    q = input.new_empty(input.shape, dtype=torch.float8_e4m3fn)
    s = torch.empty_like(input, memory_format=torch.contiguous_format) if residual is not None else input.new_empty((0,))
    row_scale = input.new_empty((0,), dtype=torch.float32) if scale_in is not None else _stat(input)
    return q, s, row_scale, input.new_empty((1,), dtype=torch.float32)


@torch.library.register_fake("fused_layernorm::norm_mxfp8")
def _(kind, input, residual, gamma, beta, epsilon):
    q = input.new_empty(input.shape, dtype=torch.float8_e4m3fn)
    s = torch.empty_like(input, memory_format=torch.contiguous_format) if residual is not None else input.new_empty((0,))
    scales = input.new_empty((input.shape[0], input.shape[1] // 32), dtype=torch.uint8)
    return q, s, scales, input.new_empty((1,), dtype=torch.float32)


@torch.library.register_fake("fused_layernorm::layernorm_bwd")
def _(grad_output, input, mean, rstd, gamma, dres_in, need_dx, need_dgamma, need_dbeta):
    cols = input.shape[1]
    dx = torch.empty_like(input, memory_format=torch.contiguous_format) if (need_dx or dres_in is not None) \
        else input.new_empty((0,))
    return dx, input.new_empty((cols if need_dgamma else 0,)), input.new_empty((cols if need_dbeta else 0,))


@torch.library.register_fake("fused_layernorm::rmsnorm_bwd")
def _(grad_output, input, rstd, gamma, dres_in, need_dx, need_dgamma):
    cols = input.shape[1]
    dx = torch.empty_like(input, memory_format=torch.contiguous_format) if (need_dx or dres_in is not None) \
        else input.new_empty((0,))
    return dx, input.new_empty((cols if need_dgamma else 0,))


@torch.library.register_fake("fused_layernorm::layernorm_bwd_f32")
def _(grad_output, input, mean, rstd, gamma):
    return torch.empty_like(input, memory_format=torch.contiguous_format), \
        input.new_empty((2 * input.shape[1],), dtype=torch.float32)


@torch.library.register_fake("fused_layernorm::cast_from_f32")
def _(src, dtype):
    return src.new_empty(src.shape, dtype=dtype)


# --------------------------------------------------------------------------------- autograd
# Gradients flow through y (and through the residual sum for the fused-add forms); the saved
# statistics are not differentiable outputs.
def _ln_setup(ctx, inputs, output):
    input, gamma, beta, _eps = inputs
    _y, mean, rstd = output
    ctx.save_for_backward(input, gamma, mean, rstd)
    ctx.has_beta = beta is not None
    ctx.set_materialize_grads(False)


def _ln_backward(ctx, gy, _gmean, _grstd):
    input, gamma, mean, rstd = ctx.saved_tensors
    if gy is None:
        return None, None, None, None
    need = ctx.needs_input_grad
    dx, dg, db = ops.layernorm_bwd(gy, input, mean, rstd, gamma, None, need[0], need[1] and gamma is not None,
                                   need[2] and ctx.has_beta)
    return _none_if_empty(dx), _none_if_empty(dg), _none_if_empty(db), None


torch.library.register_autograd("fused_layernorm::layernorm_fwd", _ln_backward, setup_context=_ln_setup)


def _rms_setup(ctx, inputs, output):
    input, gamma, _eps = inputs
    _y, rstd = output
    ctx.save_for_backward(input, gamma, rstd)
    ctx.set_materialize_grads(False)


def _rms_backward(ctx, gy, _grstd):
    input, gamma, rstd = ctx.saved_tensors
    if gy is None:
        return None, None, None
    need = ctx.needs_input_grad
    dx, dg = ops.rmsnorm_bwd(gy, input, rstd, gamma, None, need[0], need[1] and gamma is not None)
    return _none_if_empty(dx), _none_if_empty(dg), None


torch.library.register_autograd("fused_layernorm::rmsnorm_fwd", _rms_backward, setup_context=_rms_setup)


def _addln_setup(ctx, inputs, output):
    _input, _residual, gamma, beta, _eps = inputs
    _y, s, mean, rstd = output
    ctx.save_for_backward(s, gamma, mean, rstd)
    ctx.has_beta = beta is not None
    ctx.set_materialize_grads(False)


def _addln_backward(ctx, gy, gsum, _gmean, _grstd):
    s, gamma, mean, rstd = ctx.saved_tensors
    need = ctx.needs_input_grad
    if gy is None:
        d = gsum
        return (d if need[0] else None), (d if need[1] else None), None, None, None
    want_dx = need[0] or need[1]
    dx, dg, db = ops.layernorm_bwd(gy, s, mean, rstd, gamma, gsum if want_dx else None, want_dx,
                                   need[2] and gamma is not None, need[3] and ctx.has_beta)
    dx = _none_if_empty(dx)
    return (dx if need[0] else None), (dx if need[1] else None), _none_if_empty(dg), _none_if_empty(db), None


torch.library.register_autograd("fused_layernorm::add_layernorm_fwd", _addln_backward, setup_context=_addln_setup)


def _addrms_setup(ctx, inputs, output):
    _input, _residual, gamma, _eps = inputs
    _y, s, rstd = output
    ctx.save_for_backward(s, gamma, rstd)
    ctx.set_materialize_grads(False)


def _addrms_backward(ctx, gy, gsum, _grstd):
    s, gamma, rstd = ctx.saved_tensors
    need = ctx.needs_input_grad
    if gy is None:
        d = gsum
        return (d if need[0] else None), (d if need[1] else None), None, None
    want_dx = need[0] or need[1]
    dx, dg = ops.rmsnorm_bwd(gy, s, rstd, gamma, gsum if want_dx else None, want_dx, need[2] and gamma is not None)
    dx = _none_if_empty(dx)
    return (dx if need[0] else None), (dx if need[1] else None), _none_if_empty(dg), None


torch.library.register_autograd("fused_layernorm::add_rmsnorm_fwd", _addrms_backward, setup_context=_addrms_setup)


# ------------------------------------------------------------------ convenience operators
# Value-only forms of the operators above, under the names a caller would look for first.
# They are composites (CompositeImplicitAutograd): under tracing they decompose into the
# *_fwd / norm_fp8 operators, whose fakes and autograd formulas then apply, so they need none
# of their own.
_frag = torch.library.Library("fused_layernorm", "FRAGMENT")
_frag.define("rmsnorm(Tensor input, Tensor? gamma, float epsilon) -> Tensor")
_frag.define("add_layernorm(Tensor input, Tensor residual, Tensor? gamma, Tensor? beta, float epsilon) -> (Tensor, Tensor)")
_frag.define("add_rmsnorm(Tensor input, Tensor residual, Tensor? gamma, float epsilon) -> (Tensor, Tensor)")
_frag.define("add_rmsnorm_fp8(Tensor input, Tensor residual, Tensor? gamma, float epsilon) -> (Tensor, Tensor, Tensor)")


def _rmsnorm(input, gamma, epsilon):
    return ops.rmsnorm_fwd(input, gamma, epsilon)[0]


def _add_layernorm(input, residual, gamma, beta, epsilon):
    y, s, _mean, _rstd = ops.add_layernorm_fwd(input, residual, gamma, beta, epsilon)
    return y, s


def _add_rmsnorm(input, residual, gamma, epsilon):
    y, s, _rstd = ops.add_rmsnorm_fwd(input, residual, gamma, epsilon)
    return y, s


def _add_rmsnorm_fp8(input, residual, gamma, epsilon):
    """(q, sum, scale): e4m3 output with the per-tensor scale 448 / amax computed on the device."""
    q, s, scale, _mean, _rstd = ops.norm_fp8(RMSNORM, input, residual, gamma, None, epsilon)
    return q, s, scale


_frag.impl("rmsnorm", _rmsnorm, "CompositeImplicitAutograd")
_frag.impl("add_layernorm", _add_layernorm, "CompositeImplicitAutograd")
_frag.impl("add_rmsnorm", _add_rmsnorm, "CompositeImplicitAutograd")
_frag.impl("add_rmsnorm_fp8", _add_rmsnorm_fp8, "CompositeImplicitAutograd")


# ----------------------------------------------------- fused dropout -> add -> norm (C ABI)
# These two operators are defined here, in Python, on top of the C ABI (the allocation is
# torch's, the launch goes through ctypes on the current stream); the kernels are
# fln_dropout_add_norm_forward / fln_dropout_backward.
from typing import Optional, Tuple  # noqa: E402

from . import _capi  # noqa: E402


@torch.library.custom_op("fused_layernorm::dropout_add_norm_fwd", mutates_args=())
def dropout_add_norm_fwd(kind: int, input: torch.Tensor, residual: Optional[torch.Tensor], gamma: Optional[torch.Tensor],
                         beta: Optional[torch.Tensor], p: float, epsilon: float, seed: int,
                         offset: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(y, sum, mean, rstd, keep_bits) of y = norm(dropout(input, p) + residual); mean is empty for
    RMSNorm; keep_bits is uint8 [rows * cols / 8]."""
    if input.dim() != 2 or not input.is_cuda:
        raise RuntimeError("dropout_add_norm_fwd expects a 2-D CUDA tensor")
    x = input.contiguous()
    res = residual.contiguous() if residual is not None else None
    rows, cols = x.shape
    y = torch.empty_like(x)
    s = torch.empty_like(x)
    mean = x.new_empty((rows if kind == LAYERNORM else 0,), dtype=torch.float32)
    rstd = x.new_empty((rows,), dtype=torch.float32)
    bits = x.new_empty((rows * cols // 8,), dtype=torch.uint8)
    with torch.cuda.device(x.device):
        _capi.dropout_add_norm_forward(kind, x, res, gamma, beta, y, s, mean if kind == LAYERNORM else None, rstd, bits,
                                       epsilon, p, seed, offset)
    return y, s, mean, rstd, bits


@dropout_add_norm_fwd.register_fake
def _(kind, input, residual, gamma, beta, p, epsilon, seed, offset):
    e = lambda: torch.empty_like(input, memory_format=torch.contiguous_format)
    rows, cols = input.shape
    return (e(), e(), input.new_empty((rows if kind == LAYERNORM else 0,), dtype=torch.float32), _stat(input),
            input.new_empty((rows * cols // 8,), dtype=torch.uint8))


@torch.library.custom_op("fused_layernorm::dropout_bwd", mutates_args=())
def dropout_bwd(d_sum: torch.Tensor, keep_bits: torch.Tensor, p: float) -> torch.Tensor:
    """Gradient of dropout's input from the gradient of its output and the stored keep bits."""
    g = d_sum.contiguous()
    out = torch.empty_like(g)
    with torch.cuda.device(g.device):
        _capi.dropout_backward(g, keep_bits, out, p, 0, 0)
    return out


@dropout_bwd.register_fake
def _(d_sum, keep_bits, p):
    return torch.empty_like(d_sum, memory_format=torch.contiguous_format)


def _dan_setup(ctx, inputs, output):
    kind, _input, residual, gamma, beta, p, _eps, _seed, _offset = inputs
    _y, s, mean, rstd, bits = output
    ctx.save_for_backward(s, gamma, mean, rstd, bits)
    ctx.kind, ctx.p = kind, p
    ctx.has_beta = beta is not None
    ctx.has_res = residual is not None
    ctx.set_materialize_grads(False)


def _dan_backward(ctx, gy, gsum, _gmean, _grstd, _gbits):
    s, gamma, mean, rstd, bits = ctx.saved_tensors
    need = ctx.needs_input_grad  # kind, input, residual, gamma, beta, ...
    want_ds = need[1] or need[2]
    dgamma = dbeta = None
    if gy is None:
        ds = gsum
    elif ctx.kind == LAYERNORM:
        ds, dgamma, dbeta = ops.layernorm_bwd(gy, s, mean, rstd, gamma, gsum if want_ds else None, want_ds,
                                              need[3] and gamma is not None, need[4] and ctx.has_beta)
    else:
        ds, dgamma = ops.rmsnorm_bwd(gy, s, rstd, gamma, gsum if want_ds else None, want_ds, need[3] and gamma is not None)
    ds = _none_if_empty(ds)
    dx = ops.dropout_bwd(ds, bits, ctx.p) if (need[1] and ds is not None) else None
    return (None, dx, ds if (need[2] and ctx.has_res) else None, _none_if_empty(dgamma), _none_if_empty(dbeta),
            None, None, None, None)


torch.library.register_autograd("fused_layernorm::dropout_add_norm_fwd", _dan_backward, setup_context=_dan_setup)


@torch.library.custom_op("fused_layernorm::norm_nvfp4", mutates_args=())
def norm_nvfp4(kind: int, input: torch.Tensor, residual: Optional[torch.Tensor], gamma: Optional[torch.Tensor],
               beta: Optional[torch.Tensor], tensor_scale: torch.Tensor,
               epsilon: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(q, sum, block_scales, amax): NVFP4-style output of norm(input + residual) -- q uint8
    [rows, cols / 2] (two e2m1 codes per byte), block_scales uint8 [rows, cols / 16] (e4m3),
    amax fp32 [1] of this call; sum is empty without a residual.  Forward only."""
    if input.dim() != 2 or not input.is_cuda:
        raise RuntimeError("norm_nvfp4 expects a 2-D CUDA tensor")
    x = input.contiguous()
    res = residual.contiguous() if residual is not None else None
    rows, cols = x.shape
    q = x.new_empty((rows, cols // 2), dtype=torch.uint8)
    bs = x.new_empty((rows, cols // 16), dtype=torch.uint8)
    s = torch.empty_like(x) if res is not None else x.new_empty((0,))
    amax = x.new_zeros((1,), dtype=torch.float32)
    with torch.cuda.device(x.device):
        _capi.norm_forward_nvfp4(kind, x, res, gamma, beta, q, bs, s if res is not None else None, None, None,
                                 tensor_scale, amax, epsilon)
    return q, s, bs, amax


@norm_nvfp4.register_fake
def _(kind, input, residual, gamma, beta, tensor_scale, epsilon):
    rows, cols = input.shape
    s = torch.empty_like(input, memory_format=torch.contiguous_format) if residual is not None else input.new_empty((0,))
    return (input.new_empty((rows, cols // 2), dtype=torch.uint8), s,
            input.new_empty((rows, cols // 16), dtype=torch.uint8), input.new_empty((1,), dtype=torch.float32))
