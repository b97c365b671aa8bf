"""Host-side behaviour of the Python package, checked without a GPU: API surface, module
construction and state_dict compatibility, argument errors, utilities, operator schemas and
fake-tensor tracing, shard arithmetic."""
import math

import pytest
import torch
import torch.nn as nn

import fused_layernorm
import fused_layernorm_cuda
from fused_layernorm import FusedLayerNorm, FusedLayerNormFunction, FusedRMSNorm, fused_layer_norm
from fused_layernorm import functional as FF
from fused_layernorm.sharded import shard_bounds


def test_reference_surface_is_present():
    # fused_layernorm/__init__.py:14-20 of the reference
    for name in ["FusedLayerNorm", "FusedLayerNormFunction", "fused_layer_norm", "replace_torch_layernorm",
                 "restore_torch_layernorm"]:
        assert name in fused_layernorm.__all__ and hasattr(fused_layernorm, name)
    assert fused_layernorm.__version__ == "1.0.0"
    # csrc/bindings.cpp:41-44 and csrc/layernorm_cuda.cpp:198-238 of the reference
    for name in ["layernorm", "layernorm_gelu", "forward", "backward", "get_memory_usage", "get_performance_hints",
                 "__version__", "__cuda_version__"]:
        assert hasattr(fused_layernorm_cuda, name)
    assert FF.FusedLayerNormFunction is FusedLayerNormFunction
    for name in ["check_input_dtype_and_device", "get_optimal_config", "benchmark_config", "LayerNormProfiler",
                 "enable_profiling", "disable_profiling", "get_profiler"]:
        assert hasattr(FF, name)


def test_module_matches_nn_layernorm_interface():
    m = FusedLayerNorm(768)
    ref = nn.LayerNorm(768)
    assert m.normalized_shape == (768,) and m.eps == 1e-5 and m.elementwise_affine
    assert set(m.state_dict()) == set(ref.state_dict()) == {"weight", "bias"}
    assert torch.equal(m.weight, torch.ones(768)) and torch.equal(m.bias, torch.zeros(768))
    ref.weight.data.normal_()
    m.load_state_dict(ref.state_dict())
    assert torch.equal(m.weight, ref.weight)
    assert m.extra_repr() == ref.extra_repr()
    na = FusedLayerNorm((4, 8), eps=1e-6, elementwise_affine=False)
    assert na.weight is None and na.bias is None and na.normalized_shape == (4, 8)
    assert FusedLayerNorm(16, dtype=torch.bfloat16).weight.dtype == torch.bfloat16
    b, h = 32, 768
    assert m.estimate_memory_usage(b) == 2 * b * h * 4 + 2 * b * 4 + b * h * 4 + 2 * h * 4 + b * 32 * 4
    assert "Small batch" in m.get_performance_hints((2, 768))
    assert m.get_performance_hints((5,)) == "Unable to analyze performance for given input shape"


def test_argument_errors():
    x = torch.randn(4, 8)
    with pytest.raises(ValueError, match="Expected 2D input"):
        FusedLayerNormFunction.apply(torch.randn(2, 4, 8), (8,), None, None, 1e-5)
    with pytest.raises(ValueError, match="doesn't match input shape"):
        FusedLayerNormFunction.apply(x, (4,), None, None, 1e-5)
    # no CPU fallback anywhere
    with pytest.raises(RuntimeError, match="CUDA"):
        FusedLayerNorm(8)(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_layer_norm(torch.randn(2, 3, 4, 8), (8,))
    with pytest.raises(RuntimeError, match="CUDA"):
        FusedRMSNorm(8)(x)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fused_layernorm_cuda.layernorm(x, None, None, 1e-5)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fused_layernorm_cuda.forward(x)
    with pytest.raises(ValueError):
        fused_layer_norm(torch.randn(2, 8), (4,))


def test_validation_helper_messages():
    x = torch.randn(2, 4)
    with pytest.raises(RuntimeError, match="FusedLayerNorm requires CUDA tensors"):
        FF.check_input_dtype_and_device(x)


def test_profiler_and_config():
    p = FF.LayerNormProfiler()
    assert p.stop() == {}
    p.start()
    p.record(32, 768, 1.0, 2.0)
    p.record(32, 768, 3.0, 4.0)
    r = p.stop()
    assert r["num_calls"] == 2 and r["forward"]["mean_ms"] == 2.0 and r["total"]["max_ms"] == 7.0
    assert FF.get_profiler() is FF.get_profiler()
    FF.enable_profiling()
    FF.get_profiler().record(1, 2, 0.5, 0.5)
    assert FF.disable_profiling()["num_calls"] == 1
    cfg = FF.get_optimal_config(16384, 8192, torch.bfloat16)
    assert cfg["use_vectorized_load"] and cfg["use_mixed_precision"] and not cfg["use_tensor_cores"]
    assert cfg["forward"]["vec_elems"] == 8
    with pytest.raises(NotImplementedError):
        FF.get_optimal_config(4, 8, torch.float64)


def test_replace_and_restore_torch_layernorm(capsys):
    orig = torch.nn.LayerNorm
    fused_layernorm.replace_torch_layernorm()
    assert torch.nn.LayerNorm is FusedLayerNorm
    fused_layernorm.restore_torch_layernorm()
    assert torch.nn.LayerNorm is orig
    out = capsys.readouterr().out
    assert "Successfully replaced" in out and "Restored original" in out


def test_replace_layernorm_modules_shares_parameters():
    model = nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8), nn.Sequential(nn.LayerNorm(8, elementwise_affine=False)))
    w = model[1].weight
    assert fused_layernorm.replace_layernorm_modules(model) == 2
    assert isinstance(model[1], FusedLayerNorm) and model[1].weight is w
    assert isinstance(model[2][0], FusedLayerNorm) and model[2][0].weight is None


def test_layernorm_without_bias_is_constructible_and_replaceable():
    """torch.nn.LayerNorm(d, bias=False): weight only.  The module takes the same keyword, the
    module walker carries it over, and the rebound torch.nn.LayerNorm accepts it."""
    m = FusedLayerNorm(8, bias=False)
    assert m.weight is not None and m.bias is None
    assert [k for k, _ in m.named_parameters()] == ["weight"]
    m.weight.requires_grad_(False)  # a frozen weight and no bias: the inference test must not trip on None
    model = nn.Sequential(nn.LayerNorm(8, bias=False))
    w = model[0].weight
    assert fused_layernorm.replace_layernorm_modules(model) == 1
    assert model[0].weight is w and model[0].bias is None
    assert set(model.state_dict()) == {"0.weight"}
    fused_layernorm.replace_torch_layernorm()
    try:
        assert torch.nn.LayerNorm(8, bias=False).bias is None
    finally:
        fused_layernorm.restore_torch_layernorm()


def test_operator_schemas_and_fake_tracing():
    ops = torch.ops.fused_layernorm
    for name in ["layernorm", "layernorm_gelu", "layernorm_fwd", "rmsnorm_fwd", "add_layernorm_fwd", "add_rmsnorm_fwd",
                 "norm_fp8", "norm_fp8_scaled", "norm_mxfp8", "layernorm_bwd", "rmsnorm_bwd", "layernorm_bwd_f32", "cast_from_f32"]:
        assert hasattr(ops, name)
    assert "Tensor? gamma" in str(ops.layernorm_fwd.default._schema)
    # shape propagation through the fake implementations (what torch.compile relies on)
    x = torch.empty(6, 32, device="meta", dtype=torch.bfloat16)
    w = torch.empty(32, device="meta", dtype=torch.bfloat16)
    y, mean, rstd = ops.layernorm_fwd(x, w, w, 1e-5)
    assert y.shape == (6, 32) and y.dtype == torch.bfloat16 and mean.shape == (6,) and rstd.dtype == torch.float32
    dx, dg, db = ops.layernorm_bwd(y, x, mean, rstd, w, None, True, True, False)
    assert dx.shape == (6, 32) and dg.shape == (32,) and db.numel() == 0
    y2, s, r2 = ops.add_rmsnorm_fwd(x, x, w, 1e-6)
    assert s.shape == (6, 32) and r2.shape == (6,)
    q, s8, scale, m8, r8 = ops.norm_fp8(1, x, x, w, None, 1e-6)
    assert q.dtype == torch.float8_e4m3fn and scale.shape == (1,) and m8.numel() == 0
    sc = torch.empty(1, device="meta")
    q, s8, rs, amax = ops.norm_fp8_scaled(1, x, x, w, None, sc, 1e-6)  # caller's scale: no per-row scales
    assert q.dtype == torch.float8_e4m3fn and s8.shape == (6, 32) and rs.numel() == 0 and amax.shape == (1,)
    q, s8, rs, amax = ops.norm_fp8_scaled(1, x, None, w, None, None, 1e-6)
    assert rs.shape == (6,) and rs.dtype == torch.float32 and s8.numel() == 0
    q, s8, bsc, amax = ops.norm_mxfp8(1, x, x, w, None, 1e-6)
    assert q.dtype == torch.float8_e4m3fn and bsc.shape == (6, 1) and bsc.dtype == torch.uint8
    dxf, dgb = ops.layernorm_bwd_f32(y, x, mean, rstd, w)
    assert dgb.shape == (64,) and dgb.dtype == torch.float32


def test_value_only_operators_decompose_into_the_registered_forms():
    """rmsnorm, add_layernorm, add_rmsnorm, add_rmsnorm_fp8 are registered operators; on meta
    tensors they run through the fakes of the operators they are made of."""
    ops = torch.ops.fused_layernorm
    for name in ["rmsnorm", "add_layernorm", "add_rmsnorm", "add_rmsnorm_fp8"]:
        assert hasattr(ops, name)
    x = torch.empty(6, 32, device="meta", dtype=torch.bfloat16)
    w = torch.empty(32, device="meta", dtype=torch.bfloat16)
    assert ops.rmsnorm(x, w, 1e-6).shape == (6, 32)
    y, s = ops.add_layernorm(x, x, w, w, 1e-5)
    assert y.shape == s.shape == (6, 32)
    y, s = ops.add_rmsnorm(x, x, w, 1e-6)
    assert y.dtype == torch.bfloat16 and s.shape == (6, 32)
    q, s, scale = ops.add_rmsnorm_fp8(x, x, w, 1e-6)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (6, 32) and scale.shape == (1,)


def test_autograd_graph_is_built_on_fake_tensors():
    from torch._subclasses.fake_tensor import FakeTensorMode
    ops = torch.ops.fused_layernorm
    with FakeTensorMode(allow_non_fake_inputs=False):
        x = torch.empty(6, 32, dtype=torch.float32, requires_grad=True)
        w = torch.empty(32, dtype=torch.float32, requires_grad=True)
        b = torch.empty(32, dtype=torch.float32, requires_grad=True)
        y, _, _ = ops.layernorm_fwd(x, w, b, 1e-5)
        ys, s, _ = ops.add_rmsnorm_fwd(y, x, w, 1e-6)
        (ys.sum() + s.sum()).backward()
        assert x.grad.shape == (6, 32) and w.grad.shape == (32,) and b.grad.shape == (32,)


def test_shard_bounds():
    assert [shard_bounds(131072, 8, r) for r in (0, 7)] == [(0, 16384), (114688, 131072)]
    assert [shard_bounds(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [shard_bounds(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert sum(b - a for a, b in (shard_bounds(1000003, 8, r) for r in range(8))) == 1000003
    with pytest.raises(ValueError):
        shard_bounds(10, 4, 4)
