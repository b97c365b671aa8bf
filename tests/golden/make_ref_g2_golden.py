"""Generates ref_g2_b200.npz: outputs of the reference's OWN shipped CUDA kernels
(fused_layernorm_cuda.layernorm / layernorm_gelu, csrc/bindings.cpp:19-39 of the reference),
compiled unmodified for sm_100 by oracle/build_ref.py and run on a B200.

Run on a machine with a GPU, from the repository root, after `make -C oracle ref`:
    python tests/golden/make_ref_g2_golden.py [output.npz]
The committed copy is tests/golden/ref_g2_b200.npz.  Inputs are generated on the CPU from fixed
seeds and stored next to the outputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle" / "_ref"))

CASES = [("c1_32x768", 20241, 32, 768, 1.0, 0.0), ("c2_5x1023", 20242, 5, 1023, 3.0, 0.5),
         ("c2_2x4096", 20242, 2, 4096, 3.0, 0.5), ("edge_1x17", 20251, 1, 17, 1.0, 0.0),
         ("edge_13x13", 20252, 13, 13, 1.0, 0.0), ("edge_1x4097", 20253, 1, 4097, 1.0, 0.0),
         ("range_4x4096_x1000", 20254, 4, 4096, 1000.0, 0.0)]


def main():
    import ref_g2_layernorm_cuda as ref  # the reference's extension, built into oracle/_ref/
    out = {}
    for name, seed, rows, cols, scale, shift in CASES:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, cols, generator=g) * scale + shift
        gamma = 1.0 + 0.1 * torch.randn(cols, generator=g)
        beta = 0.1 * torch.randn(cols, generator=g)
        y = ref.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
        yg = ref.layernorm_gelu(x.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
        torch.cuda.synchronize()
        for k, v in (("x", x), ("gamma", gamma), ("beta", beta), ("y", y.cpu()), ("y_gelu", yg.cpu())):
            out[f"{name}/{k}"] = v.numpy()
    out["meta/device"] = np.array(torch.cuda.get_device_name(0))
    out["meta/torch"] = np.array(torch.__version__)
    dst = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "ref_g2_b200.npz"
    dst.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes on", out["meta/device"])


if __name__ == "__main__":
    main()
