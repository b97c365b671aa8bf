"""Generates tests/golden/torch_cpu_golden.npz.

The reference project holds no golden vectors: every one of its tests compares against a live
torch.nn.LayerNorm / F.layer_norm result (tests/test_layernorm.py:47-178, tests/edge_cases.py:37
of the reference).  This script freezes that ground truth for a set of small seeded cases by
running torch's CPU implementation here, so the C oracle and the CUDA kernels can be checked
against fixed numbers on a machine that has neither the reference nor the same torch build.

Run from the repository root:  python tests/golden/make_golden.py
bf16 / fp16 tensors are stored as their raw 16-bit words (uint16), fp8 as uint8 codes.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402  (only its torch_* compositions are used here)

OUT = Path(__file__).resolve().parent / "torch_cpu_golden.npz"


def raw(t):
    if t is None:
        return None
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def gen_inputs(seed, rows, cols, dtype, x_scale=1.0, x_shift=0.0, residual=False, outliers=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * x_scale + x_shift
    if outliers:
        mask = torch.rand(rows, cols, generator=g) < 0.001
        x = torch.where(mask, x * 50.0, x)
    gamma = 1.0 + 0.1 * torch.randn(cols, generator=g)
    beta = 0.1 * torch.randn(cols, generator=g)
    dy = torch.randn(rows, cols, generator=g)
    res = 0.5 * torch.randn(rows, cols, generator=g) if residual else None
    cast = lambda t: None if t is None else t.to(dtype)
    return cast(x), cast(gamma), cast(beta), cast(dy), cast(res)


CASES = [
    # name, seed, rows, cols, dtype, kind, options
    ("c1_ln_f32_32x768", 20241, 32, 768, torch.float32, "layernorm", {}),
    ("c2_ln_f32_5x1023", 20242, 5, 1023, torch.float32, "layernorm", dict(x_scale=3.0, x_shift=0.5)),
    ("c2_ln_bf16_5x1023", 20242, 5, 1023, torch.bfloat16, "layernorm", dict(x_scale=3.0, x_shift=0.5)),
    ("c2_ln_bf16_2x4096", 20242, 2, 4096, torch.bfloat16, "layernorm", dict(x_scale=3.0, x_shift=0.5)),
    ("ln_f16_8x256", 20246, 8, 256, torch.float16, "layernorm", {}),
    ("c3_addln_bf16_8x512", 20243, 8, 512, torch.bfloat16, "layernorm", dict(residual=True)),
    ("c4_addrms_fp8_bf16_8x1024", 20244, 8, 1024, torch.bfloat16, "rmsnorm",
     dict(residual=True, outliers=True, eps=1e-6, fp8=True)),
    ("rms_f32_8x384", 20247, 8, 384, torch.float32, "rmsnorm", dict(eps=1e-6)),
    ("ln_f32_noaffine_5x13", 20248, 5, 13, torch.float32, "layernorm", dict(affine=False)),
]


def main():
    out = {}
    for name, seed, rows, cols, dtype, kind, opt in CASES:
        eps = opt.get("eps", 1e-5)
        x, gamma, beta, dy, res = gen_inputs(seed, rows, cols, dtype, opt.get("x_scale", 1.0),
                                             opt.get("x_shift", 0.0), opt.get("residual", False),
                                             opt.get("outliers", False))
        if not opt.get("affine", True):
            gamma = beta = None
        if kind == "rmsnorm":
            beta = None
        fwd = O.torch_forward(x, gamma, beta, res, kind, eps, "none")
        s = fwd["sum"] if res is not None else x
        bwd = O.torch_backward(dy, s, gamma, beta, kind, eps)
        rec = {"x": raw(x), "gamma": raw(gamma), "beta": raw(beta), "dy": raw(dy), "res": raw(res),
               "y": raw(fwd["y"]), "y32": raw(fwd["y32"]), "sum": raw(fwd["sum"]),
               "mean": raw(fwd["mean"]), "rstd": raw(fwd["rstd"]),
               "dx": raw(bwd["dx"].float()), "dgamma": raw(None if bwd["dgamma"] is None else bwd["dgamma"].float()),
               "dbeta": raw(None if bwd["dbeta"] is None else bwd["dbeta"].float()),
               "eps": np.float64(eps)}
        if dtype == torch.float32:
            rec.pop("y32")  # identical to y
        if kind == "layernorm" and res is None and rows <= 8:
            rec["y_gelu_tanh"] = raw(O.torch_forward(x, gamma, beta, None, kind, eps, "gelu_tanh")["y"])
            rec["y_gelu_erf"] = raw(O.torch_forward(x, gamma, beta, None, kind, eps, "gelu_erf")["y"])
        if opt.get("fp8"):
            q, amax, scale = O.torch_quant_fp8(fwd["y32"])
            rec["q"], rec["amax"], rec["scale"] = raw(q), raw(amax), raw(scale)
        for k, v in rec.items():
            if v is not None:
                out[f"{name}/{k}"] = v
        out[f"{name}/dtype"] = np.array(str(dtype).replace("torch.", ""))
        out[f"{name}/kind"] = np.array(kind)

    # stability rows of the reference's test_numerical_stability (tests/test_layernorm.py:238-270)
    g = torch.Generator().manual_seed(20249)
    stab = torch.stack([torch.full((768,), 1e-8), torch.full((768,), 1e8),
                        torch.randn(768, generator=g) * 1e-4, torch.randn(768, generator=g) * 1e4])
    out["stability/x"] = raw(stab)
    out["stability/y"] = raw(F.layer_norm(stab, (768,), None, None, 1e-5))

    # conversion known-answers: every bf16 / fp16 / e4m3 rounding of a spread of floats
    g = torch.Generator().manual_seed(20250)
    v = torch.cat([torch.randn(1024, generator=g) * s for s in (1e-6, 1e-3, 1.0, 30.0, 400.0, 7e4)])
    v = torch.cat([v, torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10,
                                    65504.0, 65519.0, 65520.0, 6e-8, 2.0 ** -25, 2.0 ** -24])])
    out["convert/src"] = raw(v)
    out["convert/bf16"] = raw(v.to(torch.bfloat16))
    out["convert/f16"] = raw(v.to(torch.float16))
    v8 = v.clamp(-448.0, 448.0)
    out["convert/e4m3_src"] = raw(v8)
    out["convert/e4m3"] = raw(v8.to(torch.float8_e4m3fn).view(torch.uint8))
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes;", len(out), "arrays; torch", torch.__version__)


if __name__ == "__main__":
    main()
