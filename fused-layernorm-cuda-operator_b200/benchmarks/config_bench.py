#!/usr/bin/env python
"""Device-resident timings of the fused configurations beyond plain LayerNorm, through the C ABI.

  c3          residual-add + LayerNorm forward and backward, 16384 x 4096 bf16
  c3_dres     the same backward with the incoming residual-stream gradient added into dx
  c4          residual-add + RMSNorm -> fp8-e4m3 with the per-tensor scale computed in the
              kernel (two launches), 32768 x 8192 bf16
  c4_delayed  the same output in one pass with a caller-supplied scale (delayed scaling)
  c4_rowwise  the same output in one pass with one scale per row
  c4_mxfp8    the same in one pass as MXFP8 (one E8M0 scale byte per 32 elements)
  c4_nvfp4    the same in one pass as NVFP4-style 4-bit output (e2m1, one e4m3 scale per 16
              elements, caller-supplied tensor scale): 6.5625 bytes per element
  c3_dropout  dropout -> residual-add -> LayerNorm forward, 16384 x 4096 bf16, with the keep
              bits stored (8.125 bytes per element), and the dropout backward (4.125)
  dres        LayerNorm backward with incoming residual-stream gradient, 16384 x 8192 bf16

CUDA events around back-to-back launches after warm-up; every tensor is larger than the
126 MB L2.  GB/s counts each input read once and each output written once.

    python config_bench.py [--only c4_delayed] [--iters 20] [--warmup 5] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from fused_layernorm import _capi as capi  # noqa: E402

BF = torch.bfloat16


def loop_us(fn, warmup, iters):
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


def rnd(rows, cols, scale=1.0):
    return (scale * torch.randn(rows, cols, device="cuda")).to(BF)


def c3(args, with_dres):
    rows, cols = 16384, 4096
    x, r, dy = rnd(rows, cols), rnd(rows, cols, 0.5), rnd(rows, cols)
    dres = rnd(rows, cols) if with_dres else None
    g = torch.ones(cols, device="cuda", dtype=BF)
    b = torch.zeros(cols, device="cuda", dtype=BF)
    y, s, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dgb = torch.empty(2 * cols, device="cuda")
    ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, BF) // 4, 1), device="cuda")
    tf = loop_us(lambda: capi.norm_forward(capi.LAYERNORM, x, r, g, b, y, s, mean, rstd, 1e-5), args.warmup, args.iters)
    tb = loop_us(lambda: capi.norm_backward(capi.LAYERNORM, dy, s, mean, rstd, g, dres, dx, None, None, dgb, ws),
                 args.warmup, args.iters)
    n = rows * cols
    fb, bb = 8 * n, (8 if with_dres else 6) * n
    return {"shape": [rows, cols], "fwd_us": tf, "fwd_gbs": fb / tf / 1e3, "bwd_us": tb, "bwd_gbs": bb / tb / 1e3,
            "total_us": tf + tb, "total_gbs": (fb + bb) / (tf + tb) / 1e3}


def c4(args, mode):
    rows, cols = 32768, 8192
    x, r = rnd(rows, cols), rnd(rows, cols, 0.5)
    g = torch.ones(cols, device="cuda", dtype=BF)
    q = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
    s = torch.empty_like(x)
    rstd, rs = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    amax, scale = torch.zeros(1, device="cuda"), torch.ones(1, device="cuda")
    if mode == "two_phase":
        fn = lambda: capi.norm_forward_fp8(capi.RMSNORM, x, r, g, None, q, s, None, rstd, amax, scale, 1e-6)
    elif mode == "delayed":
        fn = lambda: capi.norm_forward_fp8_delayed(capi.RMSNORM, x, r, g, None, q, s, None, None, scale, amax, 1e-6)
    elif mode == "nvfp4":
        q4 = torch.empty(rows, cols // 2, dtype=torch.uint8, device="cuda")
        bs = torch.empty(rows, cols // 16, dtype=torch.uint8, device="cuda")
        ts = torch.full((1,), 448.0 * 6.0 / 8.0, device="cuda")
        fn = lambda: capi.norm_forward_nvfp4(capi.RMSNORM, x, r, g, None, q4, bs, s, None, None, ts, None, 1e-6)
        t = loop_us(fn, args.warmup, args.iters)
        return {"shape": [rows, cols], "us": t, "gbs_of_6.5625_bytes_per_element": 6.5625 * rows * cols / t / 1e3}
    elif mode == "mxfp8":
        bs = torch.empty(rows, cols // 32, dtype=torch.uint8, device="cuda")
        fn = lambda: capi.norm_forward_mxfp8(capi.RMSNORM, x, r, g, None, q, bs, s, None, None, None, 1e-6)
    else:
        fn = lambda: capi.norm_forward_fp8_rowwise(capi.RMSNORM, x, r, g, None, q, s, None, rstd, rs, None, 1e-6)
    t = loop_us(fn, args.warmup, args.iters)
    return {"shape": [rows, cols], "us": t, "gbs_of_7_bytes_per_element": 7 * rows * cols / t / 1e3}


def c3_dropout(args):
    rows, cols = 16384, 4096
    x, r, ds = rnd(rows, cols), rnd(rows, cols, 0.5), rnd(rows, cols)
    g = torch.ones(cols, device="cuda", dtype=BF)
    b = torch.zeros(cols, device="cuda", dtype=BF)
    y, s, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    bits = torch.empty(rows * cols // 8, dtype=torch.uint8, device="cuda")
    tf = loop_us(lambda: capi.dropout_add_norm_forward(capi.LAYERNORM, x, r, g, b, y, s, mean, rstd, bits, 1e-5, 0.1, 1, 0),
                 args.warmup, args.iters)
    tb = loop_us(lambda: capi.dropout_backward(ds, bits, dx, 0.1, 1, 0), args.warmup, args.iters)
    n = rows * cols
    return {"shape": [rows, cols], "fwd_us": tf, "fwd_gbs": 8.125 * n / tf / 1e3, "dropout_bwd_us": tb,
            "dropout_bwd_gbs": 4.125 * n / tb / 1e3}


def dres(args):
    rows, cols = 16384, 8192
    x, dy, dr = rnd(rows, cols), rnd(rows, cols), rnd(rows, cols)
    g = torch.ones(cols, device="cuda", dtype=BF)
    dx = torch.empty_like(x)
    mean, rstd = torch.zeros(rows, device="cuda"), torch.ones(rows, device="cuda")
    dgb = torch.empty(2 * cols, device="cuda")
    ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, BF) // 4, 1), device="cuda")
    t = loop_us(lambda: capi.norm_backward(capi.LAYERNORM, dy, x, mean, rstd, g, dr, dx, None, None, dgb, ws),
                args.warmup, args.iters)
    return {"shape": [rows, cols], "us": t, "gbs_of_8_bytes_per_element": 8 * rows * cols / t / 1e3}


CONFIGS = {
    "c3": lambda a: c3(a, False), "c3_dres": lambda a: c3(a, True),
    "c4": lambda a: c4(a, "two_phase"), "c4_delayed": lambda a: c4(a, "delayed"),
    "c4_rowwise": lambda a: c4(a, "rowwise"), "c4_mxfp8": lambda a: c4(a, "mxfp8"),
    "c4_nvfp4": lambda a: c4(a, "nvfp4"), "c3_dropout": c3_dropout, "dres": dres,
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, choices=sorted(CONFIGS))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    out = {}
    for name, fn in CONFIGS.items():
        if args.only and name != args.only:
            continue
        out[name] = fn(args)
        print(name, json.dumps({k: (round(v, 1) if isinstance(v, float) else v) for k, v in out[name].items()}), flush=True)
        torch.cuda.empty_cache()
    if args.json:
        Path(args.json).write_text(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
