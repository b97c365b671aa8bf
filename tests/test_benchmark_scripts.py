"""The report scripts under benchmarks/ keep the reference's result schema
(benchmarks/benchmark_layernorm.py:218-237, benchmarks/reproduce_speedup.py:14-86 of the
reference).  Without a GPU: they import and their column / shape tables match.  With one: a tiny
configuration runs end to end and fills every column."""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
BENCH = ROOT / "fused-layernorm-cuda-operator_b200" / "benchmarks"

# the reference's record, key for key (benchmarks/benchmark_layernorm.py:218-237)
REFERENCE_RECORD = ["model_name", "batch_size", "seq_len", "hidden_size", "total_seq_len", "dtype",
                    "pytorch_forward_ms", "fused_forward_ms", "forward_speedup", "pytorch_backward_ms",
                    "fused_backward_ms", "backward_speedup", "total_speedup", "pytorch_memory_mb", "fused_memory_mb",
                    "memory_reduction", "max_diff", "timestamp"]


def _load(name):
    spec = importlib.util.spec_from_file_location(name, BENCH / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_model_sweep_keeps_the_reference_grid_and_columns():
    ms = _load("model_sweep")
    assert ms.REFERENCE_COLUMNS == REFERENCE_RECORD
    # the reference's model table (benchmarks/benchmark_layernorm.py:30-43) and its batch / length grid (:45-58)
    assert (1600, "GPT-2 XL") in ms.MODELS and (12288, "GPT-3 175B") in ms.MODELS and len(ms.MODELS) == 12
    assert ms.BATCHES == [1, 2, 4, 8, 16, 32, 64, 128] and ms.SEQ_LENS == [128, 256, 512, 1024]


def test_hidden_size_sweep_and_config_bench_import_without_a_gpu():
    hs = _load("hidden_size_sweep")
    assert 1600 in hs.HIDDEN and 8192 in hs.HIDDEN
    cb = _load("config_bench")
    assert {"c3", "c3_dres", "c4", "c4_delayed", "c4_rowwise", "c4_mxfp8", "dres"} <= set(cb.CONFIGS)


@pytest.mark.gpu
def test_model_sweep_fills_every_column_on_a_tiny_configuration():
    ms = _load("model_sweep")
    r = ms.one_config("tiny", 256, 2, 16, "float32", warmup=1, iters=2)
    assert list(r)[:len(REFERENCE_RECORD)] == REFERENCE_RECORD
    assert r["total_seq_len"] == 32 and r["hidden_size"] == 256 and r["dtype"] == "float32"
    assert r["max_diff"] < 1e-5 and r["fused_forward_ms"] > 0 and r["fused_backward_ms"] > 0
    assert r["fused_forward_gbs"] > 0


@pytest.mark.gpu
def test_latency_table_protocols_on_one_shape():
    lt = _load("latency_table")
    # the reference's five shapes (benchmarks/reproduce_speedup.py:80-86)
    assert [(r, c) for r, c, _ in lt.SHAPES] == [(32, 768), (32, 1024), (32, 4096), (64, 4096), (17, 1023)]
    import fused_layernorm_cuda
    x = torch.randn(32, 768, device="cuda")
    w, b = torch.ones(768, device="cuda"), torch.zeros(768, device="cuda")
    fn = lambda t: fused_layernorm_cuda.layernorm(t, w, b, 1e-5)
    fresh = lt.summary(lt.fresh_tensor(fn, 32, 768, torch.float32, samples=5))
    loop = lt.summary(lt.same_tensor_loop(fn, x, repeats=2, warmup=5, iters=20))
    for s in (fresh, loop):
        assert set(s) == {"mean_us", "median_us", "cv_pct"} and s["median_us"] > 0
