#!/usr/bin/env python
"""Model-size sweep of FusedLayerNorm against torch.nn.LayerNorm on the current GPU.

Same experiment and the same result columns as the reference's
benchmarks/benchmark_layernorm.py (configurations :30-58, protocol :84-135, result record
:218-237, JSON / CSV outputs): for every (hidden size, batch, sequence length, dtype) the
forward and the forward + backward time of both modules with CUDA events around a
back-to-back loop, peak memory, the speed-ups and the largest output difference.  Added
columns: achieved GB/s of the fused forward (algorithmic bytes: input + output) and bf16.

    python model_sweep.py                       # a representative subset, about a minute
    python model_sweep.py --full                # every configuration of the reference's grid
    python model_sweep.py --out results/        # writes benchmark_results.json / .csv there
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
from datetime import datetime
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from fused_layernorm import FusedLayerNorm  # noqa: E402

MODELS = [(768, "BERT-Base"), (1024, "BERT-Large"), (768, "GPT-2 Small"), (1024, "GPT-2 Medium"),
          (1280, "GPT-2 Large"), (1600, "GPT-2 XL"), (2048, "GPT-3 Small"), (2560, "GPT-3 Medium"),
          (4096, "GPT-3 Large"), (5120, "GPT-3 XL"), (8192, "GPT-3 XXL"), (12288, "GPT-3 175B")]
BATCHES = [1, 2, 4, 8, 16, 32, 64, 128]
SEQ_LENS = [128, 256, 512, 1024]
DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
SUBSET_MODELS = {"BERT-Base", "GPT-2 XL", "GPT-3 Large", "GPT-3 XXL", "GPT-3 175B"}
SUBSET_SHAPES = [(1, 128), (8, 512), (32, 1024)]
# the columns of the reference's result record (benchmarks/benchmark_layernorm.py:218-237), in
# its order; this script's records start with them and add fused_forward_gbs
REFERENCE_COLUMNS = ["model_name", "batch_size", "seq_len", "hidden_size", "total_seq_len", "dtype",
                     "pytorch_forward_ms", "fused_forward_ms", "forward_speedup", "pytorch_backward_ms",
                     "fused_backward_ms", "backward_speedup", "total_speedup", "pytorch_memory_mb", "fused_memory_mb",
                     "memory_reduction", "max_diff", "timestamp"]


def loop_ms(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def peak_memory_mb(layer, x):
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    start = torch.cuda.memory_allocated()
    layer(x).sum().backward()
    torch.cuda.synchronize()
    return (torch.cuda.max_memory_allocated() - start) / 1e6


def one_config(model, hidden, batch, seq, dtype_name, warmup, iters):
    dtype = DTYPES[dtype_name]
    rows = batch * seq
    x = torch.randn(rows, hidden, device="cuda", dtype=dtype)
    ref = nn.LayerNorm(hidden, dtype=dtype, device="cuda")
    fused = FusedLayerNorm(hidden, dtype=dtype, device="cuda")
    fused.load_state_dict(ref.state_dict())
    xg = x.clone().requires_grad_(True)

    def step(layer):
        def run():
            xg.grad = None
            layer(xg).sum().backward()
        return run

    with torch.no_grad():
        t_ref_f = loop_ms(lambda: ref(x), warmup, iters)
        t_fus_f = loop_ms(lambda: fused(x), warmup, iters)
        diff = (ref(x).float() - fused(x).float()).abs().max().item()
    t_ref_fb = loop_ms(step(ref), warmup, iters)
    t_fus_fb = loop_ms(step(fused), warmup, iters)
    m_ref, m_fus = peak_memory_mb(ref, xg), peak_memory_mb(fused, xg)
    return {
        "model_name": model, "batch_size": batch, "seq_len": seq, "hidden_size": hidden, "total_seq_len": rows,
        "dtype": dtype_name,
        "pytorch_forward_ms": t_ref_f, "fused_forward_ms": t_fus_f, "forward_speedup": t_ref_f / t_fus_f,
        # like the reference, "backward" is the time of a forward + backward step
        "pytorch_backward_ms": t_ref_fb, "fused_backward_ms": t_fus_fb, "backward_speedup": t_ref_fb / t_fus_fb,
        "total_speedup": (t_ref_f + t_ref_fb) / (t_fus_f + t_fus_fb),
        "pytorch_memory_mb": m_ref, "fused_memory_mb": m_fus,
        "memory_reduction": 1 - m_fus / m_ref if m_ref > 0 else 0.0,
        "max_diff": diff,
        "timestamp": datetime.now().isoformat(),
        # added column, after the reference's
        "fused_forward_gbs": 2 * rows * hidden * x.element_size() / (t_fus_f * 1e-3) / 1e9,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is not available")
    print(f"GPU: {torch.cuda.get_device_name(0)}  torch {torch.__version__}  CUDA {torch.version.cuda}")
    results = []
    for hidden, model in MODELS:
        if not args.full and model not in SUBSET_MODELS:
            continue
        shapes = [(b, s) for b in BATCHES for s in SEQ_LENS] if args.full else SUBSET_SHAPES
        for batch, seq in shapes:
            for dn in args.dtypes.split(","):
                if batch * seq * hidden * DTYPES[dn].itemsize > 8e9:
                    continue
                r = one_config(model, hidden, batch, seq, dn, args.warmup, args.iters)
                results.append(r)
                print(f"{model:12s} {batch:4d}x{seq:<5d} h={hidden:<6d} {dn:9s} fwd {r['fused_forward_ms'] * 1e3:8.1f} us "
                      f"(x{r['forward_speedup']:.2f})  fwd+bwd {r['fused_backward_ms'] * 1e3:8.1f} us "
                      f"(x{r['backward_speedup']:.2f})  {r['fused_forward_gbs']:7.0f} GB/s  maxdiff {r['max_diff']:.1e}")
    geo = lambda k: float(torch.tensor([r[k] for r in results]).log().mean().exp())
    print(f"{len(results)} configurations; geometric mean speed-up: forward x{geo('forward_speedup'):.2f}, "
          f"forward+backward x{geo('backward_speedup'):.2f}")
    if args.out:
        out = Path(args.out)
        out.mkdir(parents=True, exist_ok=True)
        (out / "benchmark_results.json").write_text(json.dumps(results, indent=2))
        with open(out / "benchmark_results.csv", "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(results[0]))
            w.writeheader()
            w.writerows(results)


if __name__ == "__main__":
    main()
