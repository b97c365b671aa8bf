#!/usr/bin/env python
"""Forward and backward GB/s of LayerNorm over hidden sizes, through the C ABI, 512 MiB per tensor.

Row lengths that are powers of two, 3 / 5 / 7 times a power of two, neither (1600), and longer
than the register budget of the one-kernel backward (12288, 16384) take different launch plans;
this prints which one served each shape (`fln_describe_launch`) beside the rate, with torch's
CUDA LayerNorm forward for comparison.  GB/s counts every input read once and every output
written once (forward 2 tensors, backward 3).

    python hidden_size_sweep.py [--dtypes bfloat16,float32] [--hidden 1600,8192] [--mib 512] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from fused_layernorm import _capi as capi  # noqa: E402

HIDDEN = (768, 1024, 1280, 1600, 2048, 2560, 3072, 4096, 5120, 6144, 8192, 10240, 12288, 16384)


def loop_us(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def plan_text(d):
    if d["pipelined"]:
        return f"pipeline K={d['vecs_per_thread']} x {d['vector_bytes']}B, {d['threads_per_row']} thr/row, S={d['stages']}"
    if d["generic"]:
        return "long-row kernels"
    return f"register K={d['vecs_per_thread']}, {d['threads_per_row']} thr/row"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtypes", default="bfloat16,float32")
    ap.add_argument("--mib", type=int, default=512, help="size of each [rows, hidden] tensor")
    ap.add_argument("--json", default=None)
    ap.add_argument("--path-override", type=int, default=0,
                    help="fln_set_path_override: 0 automatic, 1 register kernels only, 2 pipeline wherever it fits")
    ap.add_argument("--skip-torch", action="store_true")
    ap.add_argument("--hidden", default=None, help="comma-separated hidden sizes instead of the built-in list")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--stages", type=int, default=0, help="fln_set_stage_override: stages per CTA of the pipelined kernels")
    args = ap.parse_args()
    capi.lib().fln_set_path_override(args.path_override)
    capi.lib().fln_set_stage_override(args.stages)
    out = []
    for dn in args.dtypes.split(","):
        dt = getattr(torch, dn)
        es = dt.itemsize
        for cols in (HIDDEN if args.hidden is None else tuple(int(h) for h in args.hidden.split(","))):
            rows = (args.mib * 1024 * 1024 // es // cols) // 64 * 64
            x = torch.randn(rows, cols, device="cuda", dtype=dt)
            dy = torch.randn_like(x)
            g = torch.ones(cols, device="cuda", dtype=dt)
            b = torch.zeros(cols, device="cuda", dtype=dt)
            y, dx = torch.empty_like(x), torch.empty_like(x)
            mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
            dg, db = torch.empty_like(g), torch.empty_like(g)
            ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, dt) // 4, 1), device="cuda")
            tf = loop_us(lambda: capi.layernorm_forward(x, g, b, y, mean, rstd, 1e-5), iters=args.iters)
            tb = loop_us(lambda: capi.layernorm_backward(dy, x, mean, rstd, g, dx, dg, db, ws), iters=args.iters)
            tt = float('inf') if args.skip_torch else loop_us(lambda: F.layer_norm(x, (cols,), g, b, 1e-5))
            nb = rows * cols * es
            rec = {"dtype": dn, "rows": rows, "hidden": cols, "fwd_us": tf, "fwd_gbs": 2 * nb / tf / 1e3,
                   "bwd_us": tb, "bwd_gbs": 3 * nb / tb / 1e3, "torch_fwd_gbs": 2 * nb / tt / 1e3,
                   "fwd_plan": plan_text(capi.describe_launch(False, rows, cols, dt)),
                   "bwd_plan": plan_text(capi.describe_launch(True, rows, cols, dt))}
            out.append(rec)
            print(f"{dn:9s} {rows:7d} x {cols:<6d} fwd {rec['fwd_gbs']:5.0f} GB/s (torch {rec['torch_fwd_gbs']:5.0f})  "
                  f"bwd {rec['bwd_gbs']:5.0f} GB/s   fwd: {rec['fwd_plan']};  bwd: {rec['bwd_plan']}", flush=True)
            del x, dy, y, dx
            torch.cuda.empty_cache()
    if args.json:
        Path(args.json).write_text(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
