"""Utilities around the fused LayerNorm, with the names of the reference's
fused_layernorm/functional.py: input validation (:13-44), get_optimal_config (:47-74),
benchmark_config (:77-129), LayerNormProfiler and its global switch (:132-213).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .layernorm import FusedLayerNormFunction  # re-exported, as the reference does (:10)
from . import _capi


def check_input_dtype_and_device(input: torch.Tensor, weight: Optional[torch.Tensor] = None,
                                 bias: Optional[torch.Tensor] = None) -> None:
    """Raise RuntimeError unless all tensors are CUDA tensors on one device with one dtype
    (same messages as the reference, functional.py:27-44)."""
    if not input.is_cuda:
        raise RuntimeError("FusedLayerNorm requires CUDA tensors")
    if weight is not None:
        if not weight.is_cuda:
            raise RuntimeError("Weight must be a CUDA tensor")
        if weight.device != input.device:
            raise RuntimeError("Weight and input must be on the same device")
        if weight.dtype != input.dtype:
            raise RuntimeError("Weight and input must have the same dtype")
    if bias is not None:
        if not bias.is_cuda:
            raise RuntimeError("Bias must be a CUDA tensor")
        if bias.device != input.device:
            raise RuntimeError("Bias and input must be on the same device")
        if bias.dtype != input.dtype:
            raise RuntimeError("Bias and input must have the same dtype")


def get_optimal_config(batch_size: int, hidden_size: int, dtype: torch.dtype = torch.float32) -> dict:
    """How a forward call of this shape is actually launched on the current device.

    Keeps the keys of the reference's advisory dict (functional.py:61-74) but fills them from
    the library's launch planner instead of rules of thumb, and adds the planner's own fields.
    """
    if dtype not in _capi.DTYPES:
        raise NotImplementedError(f'"layernorm" not implemented for {dtype}')
    fwd = _capi.describe_launch(False, batch_size, hidden_size, dtype)
    bwd = _capi.describe_launch(True, batch_size, hidden_size, dtype)
    return {
        "use_mixed_precision": dtype in (torch.float16, torch.bfloat16),
        "threads_per_block": fwd["threads_per_cta"],
        "enable_persistent_kernel": bool(fwd["pipelined"] or bwd["pipelined"] or bwd["grid"] < max(
            1, (batch_size + bwd["rows_per_cta"] - 1) // bwd["rows_per_cta"])),
        "use_vectorized_load": fwd["vec_elems"] > 1,
        "use_tensor_cores": False,  # the path is memory-bound; tensor cores are not used
        "forward": fwd,
        "backward": bwd,
    }


def benchmark_config(input_shape: Tuple[int, ...], num_iterations: int = 100, warmup_iterations: int = 10) -> dict:
    """Wall-clock forward / forward+backward timing of FusedLayerNormFunction, fp32
    (same protocol and result keys as the reference, functional.py:77-129)."""
    import time

    device = torch.cuda.current_device()
    dtype = torch.float32
    input_tensor = torch.randn(input_shape, device=device, dtype=dtype)
    rows_shape = input_tensor.reshape(-1, input_shape[-1])
    normalized_shape = (input_shape[-1],)
    weight = torch.ones(normalized_shape, device=device, dtype=dtype, requires_grad=True)
    bias = torch.zeros(normalized_shape, device=device, dtype=dtype, requires_grad=True)

    for _ in range(warmup_iterations):
        FusedLayerNormFunction.apply(rows_shape, normalized_shape, weight, bias, 1e-5)
    torch.cuda.synchronize()

    start_time = time.time()
    for _ in range(num_iterations):
        output = FusedLayerNormFunction.apply(rows_shape, normalized_shape, weight, bias, 1e-5)
    torch.cuda.synchronize()
    forward_time = (time.time() - start_time) / num_iterations * 1000  # ms

    x = rows_shape.clone().requires_grad_(True)
    grad_output = torch.randn_like(output)
    start_time = time.time()
    for _ in range(num_iterations):
        output = FusedLayerNormFunction.apply(x, normalized_shape, weight, bias, 1e-5)
        output.backward(grad_output)
    torch.cuda.synchronize()
    backward_time = (time.time() - start_time) / num_iterations * 1000  # ms

    return {
        "forward_time_ms": forward_time,
        "backward_time_ms": backward_time,
        "total_time_ms": forward_time + backward_time,
        "throughput_gb_s": (input_tensor.numel() * input_tensor.element_size() * 2) / (forward_time * 1e6),
    }


class LayerNormProfiler:
    """Collects (batch, hidden, forward ms, backward ms) records and summarizes them
    (reference functional.py:132-195)."""

    def __init__(self):
        self.profiles = []
        self.enabled = False

    def start(self):
        self.enabled = True
        self.profiles = []

    def stop(self):
        self.enabled = False
        return self.analyze_profiles()

    def record(self, batch_size: int, hidden_size: int, forward_time: float, backward_time: float):
        if self.enabled:
            self.profiles.append({
                "batch_size": batch_size,
                "hidden_size": hidden_size,
                "forward_time_ms": forward_time,
                "backward_time_ms": backward_time,
                "total_time_ms": forward_time + backward_time,
            })

    def analyze_profiles(self) -> dict:
        if not self.profiles:
            return {}
        import statistics

        def summary(values):
            return {
                "mean_ms": statistics.mean(values),
                "std_ms": statistics.stdev(values) if len(values) > 1 else 0,
                "min_ms": min(values),
                "max_ms": max(values),
            }

        return {
            "num_calls": len(self.profiles),
            "forward": summary([p["forward_time_ms"] for p in self.profiles]),
            "backward": summary([p["backward_time_ms"] for p in self.profiles]),
            "total": summary([p["total_time_ms"] for p in self.profiles]),
        }


_profiler = LayerNormProfiler()


def enable_profiling():
    """Enable global profiling of LayerNorm operations."""
    _profiler.start()


def disable_profiling():
    """Disable profiling and return results."""
    return _profiler.stop()


def get_profiler():
    """Get the global profiler instance."""
    return _profiler
