"""The reference's CPU path for the benchmarked step, timed on the host cores.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (used by bench.py's cpu_baseline leg and by
`bench.py --impl reference`).  The reference project has no CPU kernel of its own: whenever
its Python layer does not take the CUDA route it calls torch.nn.functional.layer_norm
(fused_layernorm/layernorm.py:189-193, 265-266 of the reference), and its tests define
correctness against that function.  So "the reference on CPU" is F.layer_norm forward plus its
autograd backward, run with every host thread the process may use.
"""
from __future__ import annotations

import os
import time

import torch
import torch.nn.functional as F


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def algorithmic_bytes(rows: int, cols: int, esize: int = 2, psize: int = 2) -> int:
    """Compulsory traffic of one LayerNorm forward + backward: every input read once, every
    output written once (x, y, dy, x again, dx; gamma, beta, mean, rstd, dgamma, dbeta)."""
    fwd = rows * cols * 2 * esize + 2 * cols * psize + 2 * rows * 4
    bwd = rows * cols * 3 * esize + 2 * rows * 4 + cols * psize + 2 * cols * psize
    return fwd + bwd


def make_sample(rows: int, cols: int, dtype=torch.bfloat16, seed: int = 20245):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    gamma = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    return x, dy, gamma, beta


def step(x, dy, gamma, beta, eps=1e-5):
    """One forward + backward of the reference's CPU path; returns (y, dx, dgamma, dbeta)."""
    xr = x.detach().requires_grad_(True)
    g = gamma.detach().requires_grad_(True)
    b = beta.detach().requires_grad_(True)
    y = F.layer_norm(xr, (x.shape[-1],), g, b, eps)
    y.backward(dy)
    return y.detach(), xr.grad, g.grad, b.grad


def time_steps(rows: int, cols: int, steps: int, warmup: int, dtype=torch.bfloat16, budget_s: float = 30.0):
    """Times `steps` forward+backward passes over a rows x cols sample after `warmup`
    untimed ones.  Stops early (never below one timed step) once budget_s is spent.
    Returns (seconds per step, steps actually timed, threads)."""
    n = host_threads()
    torch.set_num_threads(n)
    x, dy, gamma, beta = make_sample(rows, cols, dtype)
    for _ in range(max(warmup, 1)):
        step(x, dy, gamma, beta)
    times = []
    t_start = time.perf_counter()
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        step(x, dy, gamma, beta)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    times.sort()
    return times[len(times) // 2], len(times), n
