"""Fused LayerNorm / RMSNorm for NVIDIA B200 (sm_100a).

Drop-in for the `fused_layernorm` package of JonSnow1807/Fused-LayerNorm-CUDA-Operator
(fused_layernorm/__init__.py:7-20 of the reference exports the first five names below), with
RMSNorm, fused residual-add, fp8 output, CUDA-graph launch and row sharding added.  There is
no CPU or pure-PyTorch fallback: importing this package needs the built extension
(fused_layernorm_cuda + libfln_b200.so), and the operators need CUDA tensors.
"""
from .layernorm import (FusedLayerNorm, FusedLayerNormFunction, fused_layer_norm, replace_layernorm_modules,
                        replace_torch_layernorm, restore_torch_layernorm)
from .rmsnorm import (FusedRMSNorm, fused_add_layer_norm, fused_add_layer_norm_fp8, fused_add_norm_fp8_delayed,
                      fused_add_norm_fp8_rowwise, fused_add_norm_mxfp8, fused_add_norm_nvfp4, fused_add_rms_norm,
                      fused_add_rms_norm_fp8, fused_dropout_add_layer_norm, fused_rms_norm)

__version__ = "1.0.0"

__all__ = [
    "FusedLayerNorm",
    "FusedLayerNormFunction",
    "fused_layer_norm",
    "replace_torch_layernorm",
    "restore_torch_layernorm",
    # additions
    "replace_layernorm_modules",
    "FusedRMSNorm",
    "fused_rms_norm",
    "fused_add_layer_norm",
    "fused_add_rms_norm",
    "fused_add_rms_norm_fp8",
    "fused_add_layer_norm_fp8",
    "fused_add_norm_fp8_delayed",
    "fused_add_norm_fp8_rowwise",
    "fused_add_norm_mxfp8",
    "fused_add_norm_nvfp4",
    "fused_dropout_add_layer_norm",
]

import torch as _torch

if not _torch.cuda.is_available():
    import warnings as _warnings

    _warnings.warn("CUDA is not available. FusedLayerNorm has no CPU fallback: its operators will raise.",
                   RuntimeWarning)
