"""FusedLayerNorm: drop-in for torch.nn.LayerNorm backed by the sm_100a kernels.

Same classes, functions, argument names and error behaviour as the reference's
fused_layernorm/layernorm.py (FusedLayerNormFunction :31-109, FusedLayerNorm :112-231,
fused_layer_norm :234-266, replace_/restore_torch_layernorm :270-280), with these differences:
  * the autograd Function really has a backward kernel.  Under torch.compile it runs on the
    registered operators fused_layernorm::layernorm_fwd / layernorm_bwd (so it traces without
    graph breaks); in eager mode it calls the extension's forward / backward directly, as the
    reference does, because a registered operator with a Python autograd formula costs
    15 - 20 us of dispatch per call, more than the kernel at the latency-bound shapes;
  * inputs of any rank are handled by flattening (the reference hands rank >= 4 and
    multi-dimensional normalized_shape to F.layer_norm, :189-193, :265-266);
  * there is no CPU or pure-PyTorch fallback: CPU tensors raise, and importing this module
    without the built extension raises ImportError.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch.autograd import Function
from torch.nn import Parameter

try:
    import fused_layernorm_cuda
except ImportError as e:  # same message the reference gives (fused_layernorm/layernorm.py:22-28)
    raise ImportError(
        "Cannot import fused_layernorm_cuda. Please ensure the CUDA extension is built. "
        "Run: python build.py (in the package directory). There is no CPU fallback."
    ) from e

from . import ops as _ops  # noqa: E402  (fake + autograd registrations)

_torch_ops = torch.ops.fused_layernorm


def _require_cuda(t: torch.Tensor, name: str = "input") -> None:
    if not t.is_cuda:
        raise RuntimeError(f"FusedLayerNorm requires CUDA tensors ({name} is on {t.device}); there is no CPU fallback")


class FusedLayerNormFunction(Function):
    """Autograd function of the fused LayerNorm: apply(input, normalized_shape, weight, bias, eps).

    input must be 2-D [rows, hidden] and normalized_shape == (hidden,), as in the reference
    (fused_layernorm/layernorm.py:59-65); saves (input, weight, bias, mean, rstd) for backward
    and returns gradients for (input, None, weight, bias, None).
    """

    @staticmethod
    def forward(ctx, input: torch.Tensor, normalized_shape: Tuple[int, ...],
                weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                eps: float = 1e-5) -> torch.Tensor:
        if input.dim() != 2:
            raise ValueError(f"Expected 2D input, got {input.dim()}D")
        normalized_shape = tuple(normalized_shape)
        if len(normalized_shape) != 1 or normalized_shape[0] != input.size(1):
            raise ValueError(f"normalized_shape {normalized_shape} doesn't match input shape {input.shape}")
        _require_cuda(input)
        input = input.contiguous()
        if torch.compiler.is_compiling():
            output, mean, rstd = _torch_ops.layernorm_fwd(input, weight, bias, eps)
        else:
            output, mean, rstd = fused_layernorm_cuda.forward(input, weight, bias, eps)
        ctx.save_for_backward(input, weight, bias, mean, rstd)
        ctx.normalized_shape = normalized_shape
        ctx.eps = eps
        return output

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input, weight, bias, mean, rstd = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        needs_input_grad = ctx.needs_input_grad[0]
        needs_weight_grad = ctx.needs_input_grad[2] if weight is not None else False
        needs_bias_grad = ctx.needs_input_grad[3] if bias is not None else False
        if torch.compiler.is_compiling():
            dx, dw, db = _torch_ops.layernorm_bwd(grad_output, input, mean, rstd, weight, None, needs_input_grad,
                                                  needs_weight_grad, needs_bias_grad)
            none_if_empty = _ops._none_if_empty
            return none_if_empty(dx), None, none_if_empty(dw), none_if_empty(db), None
        dx, dw, db = fused_layernorm_cuda.backward(grad_output, input, mean, rstd, weight, bias,
                                                   [needs_input_grad, needs_weight_grad, needs_bias_grad])
        return dx, None, dw, db, None


def _apply_flat(input, normalized_shape, weight, bias, eps):
    """Normalize over the trailing len(normalized_shape) dims of an input of any rank."""
    normalized_shape = tuple(normalized_shape)
    nd = len(normalized_shape)
    if nd == 0 or tuple(input.shape[-nd:]) != normalized_shape:
        raise ValueError(f"normalized_shape {normalized_shape} doesn't match input shape {tuple(input.shape)}")
    _require_cuda(input)
    hidden = math.prod(normalized_shape)
    w = weight.reshape(hidden) if weight is not None else None
    b = bias.reshape(hidden) if bias is not None else None
    out = FusedLayerNormFunction.apply(input.reshape(-1, hidden), (hidden,), w, b, eps)
    return out.reshape(input.shape)


class FusedLayerNorm(nn.Module):
    """torch.nn.LayerNorm-compatible module (same constructor, parameter names and state_dict).

    Mirrors fused_layernorm/layernorm.py:112-231 of the reference.
    """

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True,
                 bias: bool = True, device=None, dtype=None) -> None:
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if self.elementwise_affine:
            self.weight = Parameter(torch.empty(self.normalized_shape, **factory_kwargs))
            if bias:  # torch.nn.LayerNorm(..., bias=False): weight only
                self.bias = Parameter(torch.empty(self.normalized_shape, **factory_kwargs))
            else:
                self.register_parameter("bias", None)
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.elementwise_affine:
            nn.init.ones_(self.weight)
            if self.bias is not None:
                nn.init.zeros_(self.bias)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if (input.dim() == 2 and len(self.normalized_shape) == 1 and input.is_cuda and not torch.compiler.is_compiling()
                and input.size(1) == self.normalized_shape[0] and input.is_contiguous()
                and not (torch.is_grad_enabled() and (input.requires_grad or any(
                    q is not None and q.requires_grad for q in (self.weight, self.bias))))):
            # inference: nothing to record, one call into the extension
            return fused_layernorm_cuda.layernorm(input, self.weight, self.bias, self.eps)
        if (input.dim() == 2 and len(self.normalized_shape) == 1 and input.is_cuda and not torch.compiler.is_compiling()
                and input.size(1) == self.normalized_shape[0]):
            # eager training step: forward and backward nodes both in C++
            return fused_layernorm_cuda.layernorm_autograd(input, self.weight, self.bias, self.eps)
        if input.dim() == 2 and len(self.normalized_shape) == 1:
            # direct 2-D case: the reference's fast path (layernorm.py:176-180)
            return FusedLayerNormFunction.apply(input, self.normalized_shape, self.weight, self.bias, self.eps)
        return _apply_flat(input, self.normalized_shape, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return "{normalized_shape}, eps={eps}, elementwise_affine={elementwise_affine}".format(**self.__dict__)

    @torch.jit.unused
    def estimate_memory_usage(self, batch_size: int) -> int:
        """Closed-form byte estimate of a forward+backward call (reference layernorm.py:201-214)."""
        hidden_size = math.prod(self.normalized_shape)
        use_mixed_precision = self.weight.dtype in (torch.float16, torch.bfloat16) if self.weight is not None else False
        return fused_layernorm_cuda.get_memory_usage(batch_size, hidden_size, use_mixed_precision)

    @torch.jit.unused
    def get_performance_hints(self, input_shape: Tuple[int, ...]) -> str:
        """Advisory text for an input shape (reference layernorm.py:216-231)."""
        if len(input_shape) >= 2:
            batch_size = input_shape[0] if len(input_shape) == 2 else input_shape[0] * input_shape[1]
            hidden_size = input_shape[-1]
            return fused_layernorm_cuda.get_performance_hints(batch_size, hidden_size)
        return "Unable to analyze performance for given input shape"


def fused_layer_norm(input: torch.Tensor, normalized_shape, weight: Optional[torch.Tensor] = None,
                     bias: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    """Functional form, same signature as F.layer_norm (reference layernorm.py:234-266)."""
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    normalized_shape = tuple(normalized_shape)
    if input.dim() == 2 and len(normalized_shape) == 1 and normalized_shape[0] == input.size(1):
        return FusedLayerNormFunction.apply(input, normalized_shape, weight, bias, eps)
    return _apply_flat(input, normalized_shape, weight, bias, eps)


_ORIGINAL_TORCH_LAYERNORM = torch.nn.modules.normalization.LayerNorm


def replace_torch_layernorm():
    """Rebind torch.nn.LayerNorm to FusedLayerNorm (reference layernorm.py:270-273)."""
    torch.nn.LayerNorm = FusedLayerNorm
    print("Successfully replaced torch.nn.LayerNorm with FusedLayerNorm")


def restore_torch_layernorm():
    """Undo replace_torch_layernorm (reference layernorm.py:276-280)."""
    torch.nn.LayerNorm = _ORIGINAL_TORCH_LAYERNORM
    print("Restored original torch.nn.LayerNorm")


def replace_layernorm_modules(model: nn.Module) -> int:
    """Swap every torch.nn.LayerNorm instance inside `model` for a FusedLayerNorm that shares
    its parameters (what the reference's README sketches at :103-122).  Returns the count."""
    n = 0
    for name, child in list(model.named_children()):
        if isinstance(child, _ORIGINAL_TORCH_LAYERNORM) and not isinstance(child, FusedLayerNorm):
            w = child.weight
            new = FusedLayerNorm(child.normalized_shape, child.eps, child.elementwise_affine,
                                 bias=child.bias is not None,
                                 device=w.device if w is not None else None,
                                 dtype=w.dtype if w is not None else None)
            if child.elementwise_affine:
                new.weight = child.weight
                new.bias = child.bias
            setattr(model, name, new)
            n += 1
        else:
            n += replace_layernorm_modules(child)
    return n
