#!/usr/bin/env python
"""Benchmark of the normalization hot path on B200.

One "step" = LayerNorm forward + backward over one [rows, cols] bf16 batch (default
16384 x 8192, the configuration the headline metric is quoted on), run through the library's
own multi-GPU API (`fused_layernorm.sharded.ShardedLayerNormStep`).  With N GPUs every rank
holds its own 16384-row shard (weak scaling: N = 8 is the 131072-row job) and the per-rank
[dgamma | dbeta] fp32 sums are all-reduced over NCCL each step, off the critical path.

  python bench.py [--gpus N] [--steps K] [--warmup W]            our kernels, through the C ABI
  python bench.py --impl reference ...                            the reference's CPU path
  torchrun --nproc-per-node N bench.py --gpus N ...               N > 1

Rank 0 prints ONE JSON line.  `value` is GB/s of algorithmic bytes (every input read once,
every output written once) with the batch resident in HBM; `e2e` is the same metric with the
batch in pinned host memory and all copies inside the timed region.  Besides the contract's
keys the line carries: `passes` (the K-step region repeated, with median / min / CV), `parity`
(the run checks its own outputs against float64 torch arithmetic on the GPU after the timed
region), `c5_strong` (the same step with 131072 / N rows per GPU: the row-sharded configuration
with its total fixed), `configs` (the fused configurations beyond plain LayerNorm), `roofline`,
`cpu_baseline`, `small_shape`.
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
PKG = ROOT / "fused-layernorm-cuda-operator_b200"
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(PKG))

METRIC = "layernorm_fwd_bwd_hbm_throughput"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
C5_TOTAL_ROWS = 131072

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu
# capture at the default workload (the summary under profiles/ named for that kernel and shape
# gives the command); None for any other workload
NCU_TRAFFIC = {(16384, 8192): {"bytes": 773.8e6,
                               "source": "one ncu --set full capture of norm_bwd_pipe_kernel at this workload "
                                         "(537.0 MB read + 236.8 MB written; profiles/layernorm_fwd_bwd_16384x8192_bf16.md); "
                                         "a constant of this file, not measured by this run"}}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=16384, help="rows per GPU")
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--passes", type=int, default=5, help="how often the K-step timed region is repeated")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunk-rows", type=int, default=2048, help="rows per host<->device chunk of the e2e path")
    ap.add_argument("--sm-reserve", type=int, default=-1,
                    help="SMs the persistent kernels leave free (default: 0 on one GPU, 2 when an all-reduce overlaps)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-small", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-configs", action="store_true")
    ap.add_argument("--skip-strong", action="store_true")
    ap.add_argument("--skip-parity", action="store_true")
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


def spread(xs):
    """median, min, max and coefficient of variation of a list of timings"""
    m = statistics.mean(xs)
    return {"median": statistics.median(xs), "min": min(xs), "max": max(xs),
            "cv": (statistics.pstdev(xs) / m) if m > 0 and len(xs) > 1 else 0.0, "n": len(xs)}


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


# ------------------------------------------------------------------------------------------
# the reference's CPU path (bench.py's reference arm and the cpu_baseline leg)
# ------------------------------------------------------------------------------------------
def cpu_baseline(args):
    from oracle import cpu_baseline as cb
    sec, n, threads = cb.time_steps(args.rows, args.cols, steps=10, warmup=2, budget_s=25.0)
    fwd, bwd = algorithmic_bytes(args.rows, args.cols)
    return {"value": (fwd + bwd) / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "reference",
            "sample": f"torch.nn.functional.layer_norm fwd + autograd bwd on CPU, bf16, the full {args.rows} x "
                      f"{args.cols} batch per step, median of {n} steps ({sec * 1e3:.1f} ms/step)",
            "rows_per_s": args.rows / sec}


def reference_gpu_kernel_latency():
    """us/call of the reference's own shipped CUDA kernel (its two source files compiled
    unmodified for sm_100 into oracle/_ref/ by oracle/build_ref.py), same-tensor loop of 1000
    calls after 200 warm-ups (the protocol of benchmarks/reproduce_speedup.py:46-77 of the
    reference), at the five small shapes.  None when there is no GPU or the module was not built."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        ref_dir = ROOT / "oracle" / "_ref"
        if not list(ref_dir.glob("ref_g2_layernorm_cuda*.so")):
            return None
        sys.path.insert(0, str(ref_dir))
        import ref_g2_layernorm_cuda as ref
    except Exception as e:  # the arm must still print its line
        return {"unavailable": repr(e)[:200]}
    out = {"protocol": "same-tensor loop, 200 warm-up + 1000 timed calls, best of 3, us per call, fp32",
           "kernel": "the reference's csrc/layernorm_cuda_kernel.cu built for sm_100 (oracle/_ref)"}
    for rows, cols in [(32, 768), (32, 1024), (32, 4096), (64, 4096), (17, 1023)]:
        x = torch.randn(rows, cols, device="cuda") * 3 + 0.5
        g = 1 + 0.1 * torch.randn(cols, device="cuda")
        b = 0.1 * torch.randn(cols, device="cuda")
        best = {"layernorm": float("inf"), "layernorm_gelu": float("inf")}
        for _ in range(3):
            for name, fn in (("layernorm", ref.layernorm), ("layernorm_gelu", ref.layernorm_gelu)):
                for _ in range(200):
                    fn(x, g, b, 1e-5)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(1000):
                    fn(x, g, b, 1e-5)
                e1.record()
                torch.cuda.synchronize()
                best[name] = min(best[name], e0.elapsed_time(e1))
        out[f"{rows}x{cols}_float32"] = {k: round(v, 2) for k, v in best.items()}
    return out


def run_reference(args, rank):
    """The reference's CPU path (see oracle/cpu_baseline.py), rank 0 only, on the full batch."""
    if rank != 0:
        return
    from oracle import cpu_baseline as cb
    t0 = time.perf_counter()
    sec, n, threads = cb.time_steps(args.rows, args.cols, steps=args.steps, warmup=max(args.warmup, 1), budget_s=150.0)
    fwd, bwd = algorithmic_bytes(args.rows, args.cols)
    val = (fwd + bwd) / sec / 1e9
    sample = (f"torch.nn.functional.layer_norm fwd + autograd bwd on CPU, bf16, each step the full {args.rows} rows x "
              f"{args.cols} of one GPU's batch, median of {n} timed steps")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": max(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"layernorm fwd+bwd {args.rows}x{args.cols} bf16 per GPU", "rows_per_gpu": args.rows,
                   "cols": args.cols},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_gpu = reference_gpu_kernel_latency()
    if ref_gpu is not None:
        line["reference_cuda_kernel_small_shape"] = ref_gpu
    line["wall_s"] = time.perf_counter() - t0
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# ours
# ------------------------------------------------------------------------------------------
def small_shape_latency(torch, capi):
    """us/call for the latency-bound sweep (32x768 fp32 and the 32x1024 / 32x4096 / 64x4096 /
    17x1023 shapes, fp32 and bf16), with the reference's own protocol: same-tensor back-to-back
    loop of 1000 calls after 200 warm-ups, CUDA events around the loop.  Columns: the pybind
    entry point a user of the reference calls (allocates its output), the raw C-ABI launch,
    one CUDA-graph launch per call, a graph holding 20 calls (per call), and torch's own CUDA
    LayerNorm.  A throw-away shape is timed first so that one-time costs (module import, first
    graph instantiation) do not land in the first row."""
    import torch.nn.functional as F
    import fused_layernorm_cuda as ext
    from fused_layernorm.graphs import GraphedLayerNorm
    L = capi.lib()

    def loop_us(fn, args=(), calls_per_iter=1):
        best = float("inf")
        for _ in range(3):
            for _ in range(200):
                fn(*args)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(1000):
                fn(*args)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / calls_per_iter)  # ms per 1000 iterations == us per iteration
        return best

    out = {"protocol": "same-tensor loop, 200 warm-up + 1000 timed calls, best of 3, us per call (the protocol of the "
                       "reference arm's reference_cuda_kernel_small_shape)"}
    shapes = [(48, 512, torch.float32)] + [(32, 768, torch.float32)] + \
             [(r, c, dt) for dt in (torch.float32, torch.bfloat16)
              for r, c in ((32, 1024), (32, 4096), (64, 4096), (17, 1023))]
    for n, (rows, cols, dt) in enumerate(shapes):
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
            "ours_pybind": loop_us(ext.layernorm, (x, w, b, 1e-5)),
            "ours_pybind_gelu": loop_us(ext.layernorm_gelu, (x, w, b, 1e-5)),
            "ours_c_abi": loop_us(L.fln_layernorm_forward, (px, pw, pb, py, None, None, rows, cols, code, 1e-5, st)),
            "ours_graph": loop_us(g1),
            "ours_graph_x20": loop_us(g20, (), 20),
            "ours_graph_x20_gelu": loop_us(gg, (), 20),
            "torch_cuda": loop_us(F.layer_norm, (x, (cols,), w, b, 1e-5)),
        }
        for g in (g1, g20, gg):
            g.close()
        if n == 0:
            continue  # the throw-away shape
        out[f"{rows}x{cols}_{str(dt).replace('torch.', '')}"] = {k: round(v, 2) for k, v in rec.items()}
    return out


def ulp16(torch, a, b):
    """distance in units in the last place between two bf16 tensors (sign-magnitude order)"""
    def key(t):
        i = t.view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7fff), i)
    return (key(a) - key(b)).abs()


def parity_check(torch, dist, step, x, dy, gamma, beta, eps):
    """After the timed region: this run's own outputs against float64 torch arithmetic on the
    GPU.  y / dx: 256 evenly spaced rows of this rank's shard, at most one bf16 unit in the last
    place (or 1e-5 absolute, for values that are near-zero differences).  [dgamma | dbeta]: the
    fp32 sums the step produced -- all-reduced when there are several ranks -- against float64
    column sums over every row of every rank (all-reduced in float64), with the tolerance the
    parity tests use for sums that may cancel: 1e-5 |want| + 1e-5 + 4e-7 sum|terms|."""
    rows, cols = x.shape
    g64, b64 = gamma.double(), beta.double()
    idx = torch.linspace(0, rows - 1, steps=min(256, rows), device=x.device).long()

    def stats(xs):
        mu = xs.mean(1, keepdim=True)
        var = ((xs - mu) ** 2).mean(1, keepdim=True)
        return mu, (var + eps).rsqrt()

    xs, dys = x[idx].double(), dy[idx].double()
    mu, rs = stats(xs)
    xh = (xs - mu) * rs
    y64 = xh * g64 + b64
    gg = dys * g64
    dx64 = rs * (gg - gg.mean(1, keepdim=True) - xh * (gg * xh).mean(1, keepdim=True))
    y_got, dx_got = step.y[idx], step.dx[idx]
    y_bad = (ulp16(torch, y_got, y64.to(y_got.dtype)) > 1) & ((y_got.double() - y64).abs() > 1e-5)
    dx_bad = (ulp16(torch, dx_got, dx64.to(dx_got.dtype)) > 1) & ((dx_got.double() - dx64).abs() > 1e-5)
    stat_err = max(float((step.mean[idx].double() - mu[:, 0]).abs().max()),
                   float(((step.rstd[idx].double() - rs[:, 0]).abs() / rs[:, 0]).max()))

    sums = torch.zeros(2 * cols, dtype=torch.float64, device=x.device)
    abss = torch.zeros(2 * cols, dtype=torch.float64, device=x.device)
    for a in range(0, rows, 1024):
        xs, dys = x[a:a + 1024].double(), dy[a:a + 1024].double()
        mu, rs = stats(xs)
        t = dys * ((xs - mu) * rs)
        sums[:cols] += t.sum(0)
        sums[cols:] += dys.sum(0)
        abss[:cols] += t.abs().sum(0)
        abss[cols:] += dys.abs().sum(0)
    if dist:
        dist.all_reduce(sums)
        dist.all_reduce(abss)
    got = step.last_sums_f32().double()
    tol = 1e-5 * sums.abs() + 1e-5 + 4e-7 * abss
    excess = ((got - sums).abs() - tol).max()
    dgamma, dbeta = step.finish()
    cast_bad = (ulp16(torch, torch.cat([dgamma, dbeta]), got.to(dgamma.dtype)) > 0).sum()
    flags = torch.tensor([int(y_bad.sum()), int(dx_bad.sum()), int(excess > 0), int(cast_bad)], device=x.device)
    if dist:
        dist.all_reduce(flags)
    f = flags.tolist()
    return {"ok": f == [0, 0, 0, 0] and stat_err < 1e-5, "y_rows_checked_per_rank": int(idx.numel()),
            "y_elements_beyond_1ulp": f[0], "dx_elements_beyond_1ulp": f[1], "ranks_with_param_sum_beyond_tolerance": f[2],
            "param_casts_not_exact": f[3], "max_param_sum_excess_over_tolerance": float(excess),
            "max_stat_error": stat_err,
            "reference": "float64 torch arithmetic on the GPU (no library kernel of this repository, no oracle)",
            "param_sums": "all-reduced fp32 [dgamma | dbeta] vs float64 column sums over all ranks' rows"
                          if dist else "fp32 [dgamma | dbeta] vs float64 column sums"}


def make_shard(torch, rows, cols, dt, rank, seed=20245):
    g = torch.Generator(device="cuda").manual_seed(seed + rank)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dt)
    dy = torch.randn(rows, cols, device="cuda", generator=g).to(dt)
    return x, dy


def timed_passes(torch, dist, step, x, dy, gamma, beta, K, passes, per_phase):
    """`passes` times: K steps between a barrier + synchronize on both sides, CUDA events on the
    launching stream.  per_phase=False is the timed region proper: two events, first launch to
    last (the reductions still in flight are joined inside it).  per_phase=True puts an event
    after every launch, which gives the per-kernel durations of the roofline but costs a few us
    per step (an event between two kernels keeps the second from being staged behind the
    first), so it is kept out of `value`.  Returns per pass (total ms, mean fwd ms, mean bwd ms)."""
    out = []
    for _ in range(passes):
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
        if dist:
            dist.barrier()  # last, so that every rank enters the timed region together
        torch.cuda.synchronize()
        for i in range(K):
            if per_phase or i == 0:
                ev[i][0].record()
            step.forward(x, gamma, beta)
            if per_phase:
                ev[i][1].record()
            step.backward(dy, gamma)
            if i == K - 1:
                step.finish()
            if per_phase or i == K - 1:
                ev[i][2].record()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
            torch.cuda.synchronize()
        total = ev[0][0].elapsed_time(ev[K - 1][2])
        if per_phase:
            out.append((total, statistics.mean(e[0].elapsed_time(e[1]) for e in ev),
                        statistics.mean(e[1].elapsed_time(e[2]) for e in ev)))
        else:
            out.append((total, None, None))
    return out


def max_over_ranks(torch, dist, values):
    if not dist:
        return list(values)
    t = torch.tensor(list(values), device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def fused_configs(torch):
    """Device-resident timings of the other configurations (residual-add + LayerNorm forward and
    backward, residual-add + RMSNorm with fp8 output in its four forms, backward with the
    residual-stream gradient), each with its fraction of the measured copy rate."""
    sys.path.insert(0, str(PKG / "benchmarks"))
    import config_bench as cb
    peak, src = measured_peak()
    a = argparse.Namespace(warmup=5, iters=20)
    out = {"protocol": "CUDA events around 20 back-to-back launches after 5 warm-ups; every tensor larger than L2",
           "peak_gbs": peak, "peak_source": src}
    for name, fn in cb.CONFIGS.items():
        r = fn(a)
        for k in list(r):
            if k.endswith("gbs") or "gbs_of" in k:
                r["frac_" + k] = r[k] / peak
        out[name] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}
        torch.cuda.empty_cache()
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
        # NCCL prints its version banner (NCCL_DEBUG=VERSION and up) on stdout when the first
        # communicator comes up; stdout of this script is the one JSON line, so file descriptor 1
        # points at stderr until that has happened
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    from fused_layernorm import _capi as capi
    from fused_layernorm.hostio import HostLayerNormFwdBwd
    from fused_layernorm.sharded import ShardedLayerNormStep

    # With N > 1 NCCL's all-reduce kernel runs beside the next forward; the persistent grids
    # leave a few SMs free for it (see fln_set_sm_reserve).
    sm_reserve = args.sm_reserve if args.sm_reserve >= 0 else (2 if world > 1 else 0)

    rows, cols, dt, eps = args.rows, args.cols, torch.bfloat16, 1e-5
    x, dy = make_shard(torch, rows, cols, dt, rank)
    gp = torch.Generator(device="cuda").manual_seed(20245)  # parameters identical on every rank
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=gp)).to(dt)
    beta = (0.1 * torch.randn(cols, device="cuda", generator=gp)).to(dt)
    step = ShardedLayerNormStep(rows, cols, dt, eps, sm_reserve=sm_reserve)
    step_launches = step.launches_per_step
    if world == 1:
        capi.lib().fln_set_sm_reserve(sm_reserve)

    W = max(args.warmup, 3)
    for _ in range(W):
        step.forward(x, gamma, beta)
        step.backward(dy, gamma)
    step.finish()
    torch.cuda.synchronize()

    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    plain = timed_passes(torch, dist, step, x, dy, gamma, beta, K, max(args.passes, 1), False)
    phased = timed_passes(torch, dist, step, x, dy, gamma, beta, K, max(min(args.passes, 3), 1), True)
    # the two kernels alone, back to back (K launches between two events): consecutive launches
    # overlap their tails and heads, which event-separated launches cannot
    def alone_ms(fn):
        for _ in range(3):
            fn()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            fn()
        step.finish()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / K
    fwd_alone, bwd_alone = max_over_ranks(torch, dist, [alone_ms(lambda: step.forward(x, gamma, beta)),
                                                        alone_ms(lambda: step.backward(dy, gamma))])
    clocks = sampler.stop() if rank == 0 else None
    # every pass: max over ranks; then the median pass is the reported one
    per_step = max_over_ranks(torch, dist, [p[0] / K for p in plain])
    fwd_ms = statistics.median(max_over_ranks(torch, dist, [p[1] for p in phased]))
    bwd_ms = statistics.median(max_over_ranks(torch, dist, [p[2] for p in phased]))
    instrumented_ms = statistics.median(max_over_ranks(torch, dist, [p[0] / K for p in phased]))
    ms_per_step = statistics.median(per_step)
    fwd_b, bwd_b = algorithmic_bytes(rows, cols)
    step_bytes = (fwd_b + bwd_b) * world
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    device_status = capi.lib().fln_device_status()

    parity = None
    if not args.skip_parity:
        step.forward(x, gamma, beta)
        step.backward(dy, gamma)
        step.finish()
        torch.cuda.synchronize()
        parity = parity_check(torch, dist, step, x, dy, gamma, beta, eps)
        parity["device_status"] = device_status

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
        e2e_times = []
        for _ in range(3):
            if dist:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.e2e_steps):
                pipe(xh, dyh, gamma, beta, yh, dxh, dph)
            e1.record()
            torch.cuda.synchronize()
            e2e_times.append(e0.elapsed_time(e1) / args.e2e_steps)
        e2e_times = max_over_ranks(torch, dist, e2e_times)
        e2e_ms = statistics.median(e2e_times)
        ok = bool(torch.equal(yh, step.y.cpu()) and torch.equal(dxh, step.dx.cpu()))
        e2e = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
               "ms_per_step_passes": spread(e2e_times),
               "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
               "matches_device_path": ok, "gpu_launches_per_step": pipe.launches_per_call,
               "api": "fused_layernorm.hostio.HostLayerNormFwdBwd (C ABI underneath), pinned host in/out"}
        del pipe, xh, dyh, yh, dxh

    # ---- the row-sharded configuration with its total fixed: 131072 / N rows per GPU ---------
    strong = None
    if not args.skip_strong and C5_TOTAL_ROWS % world == 0:
        srows = C5_TOTAL_ROWS // world
        del x, dy
        sstep = step if srows == rows else None
        if sstep is None:
            del step
            torch.cuda.empty_cache()
            sstep = ShardedLayerNormStep(srows, cols, dt, eps, sm_reserve=sm_reserve)
        sx, sdy = make_shard(torch, srows, cols, dt, rank, seed=30245)
        for _ in range(3):
            sstep.forward(sx, gamma, beta)
            sstep.backward(sdy, gamma)
        sstep.finish()
        torch.cuda.synchronize()
        sK = max(min(K, 20), 1)
        sp = timed_passes(torch, dist, sstep, sx, sdy, gamma, beta, sK, 3, False)
        s_per_step = max_over_ranks(torch, dist, [p[0] / sK for p in sp])
        s_ms = statistics.median(s_per_step)
        sf, sb = algorithmic_bytes(srows, cols)
        strong = {"total_rows": C5_TOTAL_ROWS, "rows_per_gpu": srows, "steps": sK, "ms_per_step": s_ms,
                  "ms_per_step_passes": spread(s_per_step),
                  "value": (sf + sb) * world / (s_ms * 1e-3) / 1e9, "unit": UNIT, "scaling": "strong",
                  "note": "same step, same API; speed-up over N = 1 is T_1 / T_N of this object's ms_per_step"}
        del sx, sdy, sstep
        torch.cuda.empty_cache()

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    bwd_gbs = bwd_b / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fwd_b / (fwd_ms * 1e-3) / 1e9
    traffic = NCU_TRAFFIC.get((rows, cols), {"bytes": None, "source": None})
    launches_per_step = step_launches
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"layernorm fwd+bwd {rows}x{cols} bf16 per GPU", "rows_per_gpu": rows, "cols": cols,
                   "total_rows": rows * world, "eps": eps, "l2": "every tensor (256 MiB) is larger than the 126 MB L2",
                   "collective": "ncclAllReduce fp32[2*cols] per step, on a side stream" if world > 1 else "none",
                   "sm_reserve": sm_reserve, "api": "fused_layernorm.sharded.ShardedLayerNormStep (C ABI underneath)"},
        "passes": {"what": f"the timed region of exactly {K} steps, repeated; ms per step of each pass (max over "
                           "ranks); ms_per_step is their median", "ms_per_step": [round(v, 6) for v in per_step],
                   **spread(per_step)},
        "rows_per_s": rows * world / (ms_per_step * 1e-3),
        "frac_of_nominal_8TBs": value / world / NOMINAL_HBM_GBS,
        "frac_of_" + peak_src: value / world / peak,
        "roofline": {"kernel": "norm_bwd_pipe_kernel (dx and the partial sums of dgamma / dbeta; their column sum "
                               "is a third, small launch on a side stream)",
                     "bound": "hbm", "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
                     "traffic": traffic["bytes"], "traffic_source": traffic["source"], "peak_source": peak_src,
                     "algorithmic_bytes": bwd_b, "avg_ms": bwd_ms, "avg_ms_back_to_back": bwd_alone,
                     "frac_back_to_back": bwd_b / (bwd_alone * 1e-3) / 1e9 / peak,
                     "timing": "avg_ms: CUDA events around every launch in further passes of the same K steps "
                               f"({instrumented_ms:.4f} ms/step with those events in the stream); "
                               "avg_ms_back_to_back: K launches of this kernel alone between two events"},
        "roofline_forward": {"kernel": "norm_fwd_pipe_kernel", "bound": "hbm", "achieved": fwd_gbs, "peak": peak,
                             "unit": "GB/s", "frac": fwd_gbs / peak, "algorithmic_bytes": fwd_b, "avg_ms": fwd_ms,
                             "avg_ms_back_to_back": fwd_alone,
                             "frac_back_to_back": fwd_b / (fwd_alone * 1e-3) / 1e9 / peak},
        "clocks": clocks, "gpu_launches": K * launches_per_step,
    }
    if parity:
        out["parity"] = parity
    if strong:
        out["c5_strong"] = strong
    if e2e:
        out["e2e"] = e2e
    if world == 1 and not args.skip_configs:
        out["configs"] = fused_configs(torch)
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
