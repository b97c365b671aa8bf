"""RMSNorm, fused residual-add + norm, and fp8-e4m3 output: the siblings of the LayerNorm path.

The reference has none of these (it ships LayerNorm and LayerNorm+GELU forward only,
csrc/bindings.cpp:41-44 of the reference); their semantics are the plain-torch compositions
    s = x + residual                      (rounded to the tensor dtype, as an unfused add would)
    y = rms_norm(s) or layer_norm(s)      (fp32 statistics, one rounding on store)
    q = (y * 448 / max|y|).to(float8_e4m3fn)
All functions take tensors of any rank and normalize over the last dimension.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch.nn import Parameter

import fused_layernorm_cuda as _ext

from . import ops as _ops  # noqa: F401
from .layernorm import _require_cuda

_t = torch.ops.fused_layernorm


def _flat(x):
    return x.reshape(-1, x.shape[-1])


def _eager() -> bool:
    """Outside torch.compile the functions below call the extension directly (its autograd nodes
    are C++); while compiling they go through the registered fused_layernorm::* operators.  A
    registered operator with a Python autograd formula costs 15 - 20 us per call in eager mode."""
    return not torch.compiler.is_compiling()


def fused_rms_norm(input: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight over the last dimension (differentiable)."""
    _require_cuda(input)
    if _eager():
        y, _s = _ext.norm_autograd(_ops.RMSNORM, _flat(input), None, weight, None, eps)
    else:
        y, _rstd = _t.rmsnorm_fwd(_flat(input), weight, eps)
    return y.reshape(input.shape)


def fused_add_layer_norm(input: torch.Tensor, residual: torch.Tensor, weight: Optional[torch.Tensor] = None,
                         bias: Optional[torch.Tensor] = None, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """(layer_norm(input + residual), input + residual) in one pass over HBM (differentiable;
    a gradient arriving on the returned sum is added into the input gradient by the kernel)."""
    _require_cuda(input)
    if _eager():
        y, s = _ext.norm_autograd(_ops.LAYERNORM, _flat(input), _flat(residual), weight, bias, eps)
    else:
        y, s, _mean, _rstd = _t.add_layernorm_fwd(_flat(input), _flat(residual), weight, bias, eps)
    return y.reshape(input.shape), s.reshape(input.shape)


def fused_add_rms_norm(input: torch.Tensor, residual: torch.Tensor, weight: Optional[torch.Tensor] = None,
                       eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """(rms_norm(input + residual), input + residual) in one pass over HBM (differentiable)."""
    _require_cuda(input)
    if _eager():
        y, s = _ext.norm_autograd(_ops.RMSNORM, _flat(input), _flat(residual), weight, None, eps)
    else:
        y, s, _rstd = _t.add_rmsnorm_fwd(_flat(input), _flat(residual), weight, eps)
    return y.reshape(input.shape), s.reshape(input.shape)


_dropout_calls = 0


def fused_dropout_add_layer_norm(input: torch.Tensor, residual: Optional[torch.Tensor] = None,
                                 weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                                 p: float = 0.1, eps: float = 1e-5, training: bool = True, rms: bool = False,
                                 seed: Optional[int] = None, offset: Optional[int] = None):
    """(norm(dropout(input, p) + residual), dropout(input, p) + residual) in one pass over HBM:
    the head of a pre-norm transformer block (differentiable in input, residual, weight, bias; a
    gradient arriving on the returned sum is added in).  `rms=True` selects RMSNorm.  With
    training=False (or p == 0) nothing is dropped.  The mask is the Philox4x32-10 mask of
    (seed, offset); by default seed is torch's CUDA seed and offset counts the calls of this
    function, so torch.manual_seed makes a run reproducible.  Needs a last dimension that is a
    multiple of 8 and at most 16384."""
    global _dropout_calls
    _require_cuda(input)
    if not training:
        p = 0.0
    if seed is None:
        seed = torch.cuda.initial_seed() & 0xffffffffffffffff
    if offset is None:
        offset = _dropout_calls
        _dropout_calls += 1
    kind = _ops.RMSNORM if rms else _ops.LAYERNORM
    res = _flat(residual) if residual is not None else None
    y, s, _mean, _rstd, _bits = _t.dropout_add_norm_fwd(kind, _flat(input), res, weight, None if rms else bias, float(p),
                                                        float(eps), int(seed), int(offset))
    return y.reshape(input.shape), s.reshape(input.shape)


def fused_add_rms_norm_fp8(input: torch.Tensor, residual: Optional[torch.Tensor] = None,
                           weight: Optional[torch.Tensor] = None, eps: float = 1e-6):
    """(q, sum, scale): q = rms_norm(input + residual) quantized to float8_e4m3fn with the
    per-tensor scale 448 / max|y| computed on the device; sum = input + residual (None when
    residual is None); scale is a 1-element fp32 tensor (dequantize with q.float() / scale).
    Forward only."""
    _require_cuda(input)
    q, s, scale, _mean, _rstd = _t.norm_fp8(_ops.RMSNORM, _flat(input), None if residual is None else _flat(residual),
                                            weight, None, eps)
    return q.reshape(input.shape), (s.reshape(input.shape) if residual is not None else None), scale


def fused_add_layer_norm_fp8(input: torch.Tensor, residual: Optional[torch.Tensor] = None,
                             weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                             eps: float = 1e-5):
    """LayerNorm variant of fused_add_rms_norm_fp8."""
    _require_cuda(input)
    q, s, scale, _mean, _rstd = _t.norm_fp8(_ops.LAYERNORM, _flat(input), None if residual is None else _flat(residual),
                                            weight, bias, eps)
    return q.reshape(input.shape), (s.reshape(input.shape) if residual is not None else None), scale


def fused_add_norm_fp8_delayed(input: torch.Tensor, scale: torch.Tensor, residual: Optional[torch.Tensor] = None,
                               weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                               eps: float = 1e-6, kind: str = "rmsnorm"):
    """(q, sum, amax) in ONE pass: q = norm(input + residual) * scale, saturated to float8_e4m3fn,
    with a scale fixed beforehand (delayed scaling: usually 448 / amax of the previous step);
    amax = max|y| of this call, for the next step's scale.  `scale` is one fp32 on the device.
    7 instead of 9 bytes per element compared with fused_add_rms_norm_fp8.  Forward only."""
    _require_cuda(input)
    k = _ops.RMSNORM if kind == "rmsnorm" else _ops.LAYERNORM
    q, s, _rs, amax = _t.norm_fp8_scaled(k, _flat(input), None if residual is None else _flat(residual), weight, bias,
                                         scale, eps)
    return q.reshape(input.shape), (s.reshape(input.shape) if residual is not None else None), amax


def fused_add_norm_fp8_rowwise(input: torch.Tensor, residual: Optional[torch.Tensor] = None,
                               weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                               eps: float = 1e-6, kind: str = "rmsnorm"):
    """(q, sum, row_scale) in ONE pass: every row is quantized with its own scale
    448 / max|y[row]| (1 for an all-zero row); dequantize with q.float() / row_scale[:, None].
    row_scale has one fp32 per row of the flattened input.  Forward only."""
    _require_cuda(input)
    k = _ops.RMSNORM if kind == "rmsnorm" else _ops.LAYERNORM
    q, s, rs, _amax = _t.norm_fp8_scaled(k, _flat(input), None if residual is None else _flat(residual), weight, bias,
                                         None, eps)
    return q.reshape(input.shape), (s.reshape(input.shape) if residual is not None else None), rs


def fused_add_norm_mxfp8(input: torch.Tensor, residual: Optional[torch.Tensor] = None,
                         weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                         eps: float = 1e-6, kind: str = "rmsnorm"):
    """(q, sum, block_scale) in ONE pass, in the OCP microscaling format MXFP8 that Blackwell's
    block-scaled matrix instructions take: q is float8_e4m3fn, and every 32 consecutive elements
    of the last dimension share one power-of-two scale, returned as E8M0 bytes of shape
    input.shape[:-1] + (hidden // 32,) (dtype float8_e8m0fnu where torch has it, else uint8).
    Dequantize with q.float() * 2 ** (byte - 127) per block.  Forward only."""
    _require_cuda(input)
    k = _ops.RMSNORM if kind == "rmsnorm" else _ops.LAYERNORM
    q, s, scales, _amax = _t.norm_mxfp8(k, _flat(input), None if residual is None else _flat(residual), weight, bias,
                                        eps)
    scales = scales.reshape(*input.shape[:-1], input.shape[-1] // 32)
    if hasattr(torch, "float8_e8m0fnu"):
        scales = scales.view(torch.float8_e8m0fnu)
    return q.reshape(input.shape), (s.reshape(input.shape) if residual is not None else None), scales


def fused_add_norm_nvfp4(input: torch.Tensor, tensor_scale: torch.Tensor, residual: Optional[torch.Tensor] = None,
                         weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, eps: float = 1e-6,
                         rms: bool = True):
    """(q, block_scales, amax, sum-or-None): one-pass NVFP4-style output of norm(input + residual):
    e2m1 codes two per byte, one e4m3 scale per 16 elements, the fp32 tensor scale supplied by
    the caller (448 * 6 / amax of the previous step); y ~ e2m1(q) * e4m3(block_scale) / tensor_scale.
    The last dimension must be a multiple of 16.  Forward only."""
    _require_cuda(input)
    kind = _ops.RMSNORM if rms else _ops.LAYERNORM
    res = _flat(residual) if residual is not None else None
    q, s, bs, amax = _t.norm_nvfp4(kind, _flat(input), res, weight, None if rms else bias, tensor_scale, float(eps))
    lead = input.shape[:-1]
    return (q.reshape(*lead, -1), bs.reshape(*lead, -1), amax, s.reshape(input.shape) if residual is not None else None)


class FusedRMSNorm(nn.Module):
    """torch.nn.RMSNorm-compatible module (normalized_shape, eps, elementwise_affine; parameter `weight`)."""

    def __init__(self, normalized_shape, eps: Optional[float] = None, elementwise_affine: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        if len(self.normalized_shape) != 1:
            raise ValueError("FusedRMSNorm normalizes over the last dimension only")
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        eps = self.eps if self.eps is not None else torch.finfo(input.dtype).eps
        return fused_rms_norm(input, self.weight, eps)

    def extra_repr(self) -> str:
        return "{normalized_shape}, eps={eps}, elementwise_affine={elementwise_affine}".format(**self.__dict__)
