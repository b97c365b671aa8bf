#!/usr/bin/env python
"""us per call of `fused_layernorm_cuda.layernorm` on the latency-bound shapes, next to
torch.nn.LayerNorm, under the reference's two protocols and a third one.

The shapes and the first two protocols are those of the reference's
benchmarks/reproduce_speedup.py (fresh tensor, one event pair per call, :14-44; same tensor,
200 warm-ups, events around 1000 back-to-back calls, :46-77; shapes :80-86).  The third
column replays a CUDA graph that holds 20 calls, which is how a launch-bound inner loop is
meant to be run here.  Prints mean, median and coefficient of variation (stable below 5 %,
the criterion of the reference's tests/stable_measurement.py:67-74) and writes JSON on request.

    python latency_table.py [--dtype float32|bfloat16] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import fused_layernorm_cuda  # noqa: E402
from fused_layernorm.graphs import GraphedLayerNorm  # noqa: E402

SHAPES = [(32, 768, "BERT"), (32, 1024, "GPT-2"), (32, 4096, "GPT-3"), (64, 4096, "Large"), (17, 1023, "Odd")]


def fresh_tensor(fn, rows, cols, dtype, samples=100):
    """A new input for every call, one event pair per call (what a cold call costs)."""
    ts = []
    for _ in range(samples):
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(x)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return ts


def same_tensor_loop(fn, x, repeats=5, warmup=200, iters=1000):
    """Back-to-back calls on one tensor; one sample = the mean of `iters` calls."""
    ts = []
    for _ in range(repeats):
        for _ in range(warmup):
            fn(x)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn(x)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / iters)
    return ts


def summary(ts):
    m = statistics.mean(ts)
    return {"mean_us": m, "median_us": statistics.median(ts),
            "cv_pct": 100 * statistics.pstdev(ts) / m if m > 0 else 0.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    dtype = getattr(torch, args.dtype)
    print(f"GPU: {torch.cuda.get_device_name(0)}  dtype {args.dtype}")
    print(f"{'shape':16s} {'protocol':18s} {'torch us':>9s} {'ours us':>9s} {'speed-up':>9s} {'cv % (ours)':>12s}")
    out = []
    for rows, cols, name in SHAPES:
        ln = nn.LayerNorm(cols, device="cuda", dtype=dtype)
        ours = lambda x: fused_layernorm_cuda.layernorm(x, ln.weight, ln.bias, 1e-5)
        theirs = lambda x: ln(x)
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        with torch.no_grad():
            rec = {"shape": [rows, cols], "name": name, "dtype": args.dtype,
                   "fresh_tensor": {"torch": summary(fresh_tensor(theirs, rows, cols, dtype)),
                                    "ours": summary(fresh_tensor(ours, rows, cols, dtype))},
                   "same_tensor_loop": {"torch": summary(same_tensor_loop(theirs, x)),
                                        "ours": summary(same_tensor_loop(ours, x))}}
            graphed = GraphedLayerNorm(x, ln.weight.detach(), ln.bias.detach(), 1e-5, repeat=20)
            g = same_tensor_loop(lambda _x: graphed(), x, iters=200)
            rec["graph_of_20_calls"] = {"ours": summary([t / 20 for t in g])}
        out.append(rec)
        label = f"{name} {rows}x{cols}"
        for proto in ("fresh_tensor", "same_tensor_loop"):
            t, o = rec[proto]["torch"], rec[proto]["ours"]
            print(f"{label:16s} {proto:18s} {t['median_us']:9.2f} {o['median_us']:9.2f} "
                  f"{t['median_us'] / o['median_us']:8.2f}x {o['cv_pct']:12.1f}")
        o = rec["graph_of_20_calls"]["ours"]
        print(f"{label:16s} {'graph_of_20_calls':18s} {'':9s} {o['median_us']:9.2f} {'':9s} {o['cv_pct']:12.1f}")
    if args.json:
        Path(args.json).write_text(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
