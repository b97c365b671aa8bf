#!/usr/bin/env python
"""Benchmark of the normalization hot path on B200.

One "step" = LayerNorm forward + backward over one [rows, cols] bf16 batch (default
16384 x 8192, the configuration the headline metric is quoted on).  With N GPUs every rank
holds its own 16384-row shard (weak scaling: N = 8 is the 131072-row job) and the per-rank
[dgamma | dbeta] fp32 partials are all-reduced over NCCL each step.

  python bench.py [--gpus N] [--steps K] [--warmup W]            our kernels, through the C ABI
  python bench.py --impl reference ...                            the reference's CPU path
  torchrun --nproc-per-node N bench.py --gpus N ...               N > 1

Rank 0 prints ONE JSON line.  `value` is GB/s of algorithmic bytes (every input read once,
every output written once) with the batch resident in HBM; `e2e` is the same metric with the
batch in pinned host memory and all copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "fused-layernorm-cuda-operator_b200"))

METRIC = "layernorm_fwd_bwd_hbm_throughput"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=16384, help="rows per GPU")
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunk-rows", type=int, default=2048, help="rows per host<->device chunk of the e2e path")
    ap.add_argument("--cpu-sample-rows", type=int, default=2048)
    ap.add_argument("--sm-reserve", type=int, default=-1,
                    help="SMs the persistent kernels leave free (default: 0 on one GPU, 2 when an all-reduce overlaps)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-small", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    return ap.parse_args()


def algorithmic_bytes(rows, cols, esize=2, psize=2):
    fwd = rows * cols * 2 * esize + 2 * cols * psize + 2 * rows * 4
    bwd = rows * cols * 3 * esize + 2 * rows * 4 + cols * psize + 2 * cols * psize
    return fwd, bwd


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(args):
    from oracle import cpu_baseline as cb
    rows = min(args.cpu_sample_rows, args.rows)
    sec, n, threads = cb.time_steps(rows, args.cols, steps=10, warmup=2, budget_s=25.0)
    fwd, bwd = algorithmic_bytes(rows, args.cols)
    return {"value": (fwd + bwd) / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "reference",
            "sample": f"torch.nn.functional.layer_norm fwd + autograd bwd on CPU, bf16, {rows} of {args.rows} rows x "
                      f"{args.cols}, median of {n} steps ({sec * 1e3:.1f} ms/step)",
            "rows_per_s": rows / sec}


def run_reference(args, rank):
    """The reference's CPU path (see oracle/cpu_baseline.py), rank 0 only."""
    if rank != 0:
        return
    from oracle import cpu_baseline as cb
    rows = min(args.cpu_sample_rows, args.rows)
    t0 = time.perf_counter()
    sec, n, threads = cb.time_steps(rows, args.cols, steps=args.steps, warmup=max(args.warmup, 1), budget_s=150.0)
    fwd, bwd = algorithmic_bytes(rows, args.cols)
    val = (fwd + bwd) / sec / 1e9
    sample = (f"torch.nn.functional.layer_norm fwd + autograd bwd on CPU, bf16, each step {rows} rows x {args.cols} "
              f"(a {rows}/{args.rows} sample of the per-GPU batch), median of {n} timed steps")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": max(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"layernorm fwd+bwd {args.rows}x{args.cols} bf16 per GPU", "rows_per_gpu": args.rows,
                   "cols": args.cols, "sample_rows": rows},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }), flush=True)


def small_shape_latency(torch, capi):
    """us/call for the latency-bound sweep (32x768 fp32 and the 32x1024 / 32x4096 / 64x4096 /
    17x1023 shapes, fp32 and bf16), with the reference's own protocol: same-tensor back-to-back
    loop of 1000 calls after 200 warm-ups, CUDA events around the loop.  Columns: the pybind
    entry point a user of the reference calls (allocates its output), the raw C-ABI launch,
    one CUDA-graph launch per call, a graph holding 20 calls (per call), and torch's own CUDA
    LayerNorm."""
    import torch.nn.functional as F
    import fused_layernorm_cuda as ext
    from fused_layernorm.graphs import GraphedLayerNorm
    L = capi.lib()

    def loop_us(fn, calls_per_iter=1):
        for _ in range(200):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(1000):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / calls_per_iter  # ms per 1000 iterations == us per iteration

    out = {"protocol": "same-tensor loop, 200 warm-up + 1000 timed calls, us per call"}
    shapes = [(32, 768, torch.float32)] + [(r, c, dt) for dt in (torch.float32, torch.bfloat16)
                                           for r, c in ((32, 1024), (32, 4096), (64, 4096), (17, 1023))]
    for rows, cols, dt in shapes:
        x = (torch.randn(rows, cols, device="cuda") * 3 + 0.5).to(dt)
        w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dt)
        b = (0.1 * torch.randn(cols, device="cuda")).to(dt)
        y = torch.empty_like(x)
        px, pw, pb, py, st = capi.ptr(x), capi.ptr(w), capi.ptr(b), capi.ptr(y), capi.stream_handle()
        code = capi.DTYPES[dt]
        g1 = GraphedLayerNorm(x, w, b, 1e-5)
        g20 = GraphedLayerNorm(x, w, b, 1e-5, repeat=20)
        gg = GraphedLayerNorm(x, w, b, 1e-5, gelu="tanh", repeat=20)
        rec = {
            "ours_pybind": loop_us(lambda: ext.layernorm(x, w, b, 1e-5)),
            "ours_pybind_gelu": loop_us(lambda: ext.layernorm_gelu(x, w, b, 1e-5)),
            "ours_c_abi": loop_us(lambda: L.fln_layernorm_forward(px, pw, pb, py, None, None, rows, cols, code, 1e-5, st)),
            "ours_graph": loop_us(lambda: g1()),
            "ours_graph_x20": loop_us(lambda: g20(), 20),
            "ours_graph_x20_gelu": loop_us(lambda: gg(), 20),
            "torch_cuda": loop_us(lambda: F.layer_norm(x, (cols,), w, b, 1e-5)),
        }
        for g in (g1, g20, gg):
            g.close()
        out[f"{rows}x{cols}_{str(dt).replace('torch.', '')}"] = {k: round(v, 2) for k, v in rec.items()}
    return out


def run_ours(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with --nproc-per-node {args.gpus} (WORLD_SIZE={world})")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from fused_layernorm import _capi as capi
    from fused_layernorm.hostio import HostLayerNormFwdBwd

    # With N > 1 NCCL's all-reduce kernel runs beside the next forward; the persistent grids
    # leave a few SMs free for it (see fln_set_sm_reserve).
    sm_reserve = args.sm_reserve if args.sm_reserve >= 0 else (2 if world > 1 else 0)
    capi.lib().fln_set_sm_reserve(sm_reserve)

    rows, cols, dt = args.rows, args.cols, torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(20245 + rank)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dt)
    dy = torch.randn(rows, cols, device="cuda", generator=g).to(dt)
    gp = torch.Generator(device="cuda").manual_seed(20245)  # parameters identical on every rank
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=gp)).to(dt)
    beta = (0.1 * torch.randn(cols, device="cuda", generator=gp)).to(dt)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    dgb = torch.empty(2 * cols, device="cuda")
    dparams = torch.empty(2 * cols, dtype=dt, device="cuda")
    ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, dt) // 4, 1), device="cuda")
    # forward, backward (the column reduce is the tail of the same cooperative launch) (+ cast)
    launches_per_step = 2 + (1 if world > 1 else 0)

    # N > 1: the all-reduce of the fp32 [dgamma | dbeta] partials and the rounding to bf16 run on
    # a side stream, gated by an event behind the backward, so they overlap the next step and
    # the main stream never waits for them (a training loop needs the parameter gradients only
    # at its optimizer step).  Two buffers alternate; before a buffer is written again the main
    # stream waits for the event that marks its previous reduction as finished, which by then
    # lies a whole step in the past.  The last reductions are joined inside the timed region.
    dgb2 = [dgb, torch.empty_like(dgb)]
    side = torch.cuda.Stream() if world > 1 else None
    ev_bwd = [torch.cuda.Event() for _ in range(2)]
    ev_red = [torch.cuda.Event() for _ in range(2)]
    step_no = [0]

    def fwd():
        capi.layernorm_forward(x, gamma, beta, y, mean, rstd, 1e-5)

    def finish_pending():
        if world > 1:
            torch.cuda.current_stream().wait_stream(side)

    def bwd():
        if world > 1:
            k = step_no[0] & 1
            buf = dgb2[k]
            main = torch.cuda.current_stream()
            if step_no[0] >= 2:
                main.wait_event(ev_red[k])
            step_no[0] += 1
            capi.norm_backward(capi.LAYERNORM, dy, x, mean, rstd, gamma, None, dx, None, None, buf, ws)
            ev_bwd[k].record(main)
            with torch.cuda.stream(side):
                side.wait_event(ev_bwd[k])
                dist.all_reduce(buf)
                capi.cast_from_f32(buf, dparams, stream=side)
                ev_red[k].record(side)
        else:
            capi.norm_backward(capi.LAYERNORM, dy, x, mean, rstd, gamma, None, dx, dparams[:cols], dparams[cols:],
                               None, ws)

    for _ in range(max(args.warmup, 3)):
        fwd()
        bwd()
    if world > 1:
        finish_pending()
    torch.cuda.synchronize()

    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)

    def timed_pass(per_phase):
        """K steps between a barrier + synchronize on both sides.  per_phase=False is the
        timed region proper: two events, first launch to last.  per_phase=True repeats the
        same K steps with an event after every phase, which gives the per-kernel launch
        durations of the roofline but costs a few us per step (an event between two kernels
        keeps the second from being staged behind the first), so it is kept out of `value`."""
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
        # the barrier comes last, so every rank enters the timed region together
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        for i in range(K):
            if per_phase or i == 0:
                ev[i][0].record()
            fwd()
            if per_phase:
                ev[i][1].record()
            bwd()
            if world > 1 and i == K - 1:
                finish_pending()
            if per_phase or i == K - 1:
                ev[i][2].record()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
            torch.cuda.synchronize()
        return ev

    ev = timed_pass(False)
    total_ms = ev[0][0].elapsed_time(ev[K - 1][2])
    ev = timed_pass(True)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    instrumented_ms = ev[0][0].elapsed_time(ev[K - 1][2]) / K
    clocks = sampler.stop() if rank == 0 else None
    if dist:
        t = torch.tensor([total_ms, fwd_ms, bwd_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, fwd_ms, bwd_ms = t.tolist()
    ms_per_step = total_ms / K
    fwd_b, bwd_b = algorithmic_bytes(rows, cols)
    step_bytes = (fwd_b + bwd_b) * world
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: batch in pinned host memory, copies inside the timed region ----------
    e2e = None
    if not args.skip_e2e:
        pipe = HostLayerNormFwdBwd(rows, cols, dt, chunk_rows=args.e2e_chunk_rows)
        xh, dyh = x.cpu().pin_memory(), dy.cpu().pin_memory()
        yh, dxh = torch.empty_like(xh).pin_memory(), torch.empty_like(xh).pin_memory()
        dph = torch.empty(2 * cols, dtype=dt).pin_memory()
        for _ in range(2):
            pipe(xh, dyh, gamma, beta, yh, dxh, dph)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            pipe(xh, dyh, gamma, beta, yh, dxh, dph)
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
        if dist:
            t = torch.tensor([e2e_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t[0])
        ok = bool(torch.equal(yh, y.cpu()) and torch.equal(dxh, dx.cpu()))
        e2e = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
               "matches_device_path": ok, "gpu_launches_per_step": pipe.launches_per_call,
               "api": "fused_layernorm.hostio.HostLayerNormFwdBwd (C ABI underneath), pinned host in/out"}
        del pipe, xh, dyh, yh, dxh

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    bwd_gbs = bwd_b / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fwd_b / (fwd_ms * 1e-3) / 1e9
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"layernorm fwd+bwd {rows}x{cols} bf16 per GPU", "rows_per_gpu": rows, "cols": cols,
                   "total_rows": rows * world, "eps": 1e-5, "l2": "every tensor (256 MiB) is larger than the 126 MB L2",
                   "collective": "ncclAllReduce fp32[2*cols] per step" if world > 1 else "none",
                   "sm_reserve": sm_reserve},
        "rows_per_s": rows * world / (ms_per_step * 1e-3),
        "frac_of_nominal_8TBs": value / world / NOMINAL_HBM_GBS,
        "frac_of_" + peak_src: value / world / peak,
        "roofline": {"kernel": "norm_bwd_pipe_kernel (dx, partial sums and the fused column reduce, one launch)", "bound": "hbm", "achieved": bwd_gbs,
                     "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this launch
                     # (profiles/layernorm_fwd_bwd_16384x8192_bf16.md); only for the default workload
                     "traffic": 769.2e6 if (rows, cols) == (16384, 8192) else None, "peak_source": peak_src,
                     "algorithmic_bytes": bwd_b, "avg_ms": bwd_ms,
                     "timing": "CUDA events around every launch in a second pass of the same K steps "
                               f"({instrumented_ms:.4f} ms/step with those events in the stream)"},
        "roofline_forward": {"kernel": "norm_fwd_pipe_kernel", "bound": "hbm", "achieved": fwd_gbs, "peak": peak,
                             "unit": "GB/s", "frac": fwd_gbs / peak, "algorithmic_bytes": fwd_b, "avg_ms": fwd_ms},
        "clocks": clocks, "gpu_launches": K * launches_per_step,
    }
    if e2e:
        out["e2e"] = e2e
    if not args.skip_small and world == 1:
        out["small_shape"] = small_shape_latency(torch, capi)
    if not args.skip_cpu and world == 1:
        out["cpu_baseline"] = cpu_baseline(args)
    print(json.dumps(out), flush=True)
    if dist:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
