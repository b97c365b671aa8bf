"""CUDA-graph launch path for latency-bound shapes.

At the reference's README shapes (32 x 768 ... 64 x 4096) the kernel runs for a few
microseconds and what a caller measures is host work: argument parsing, allocation, launch
(the reference's own numbers are ~10 us per call whatever the shape,
publication_validation_results.json:91-171 of the reference).  Recording the launches once and
replaying them removes that host work.  Two routes are offered:

  * GraphedLayerNorm / GraphedLayerNormStep: static buffers, recorded through the C ABI's own
    graph entry points (fln_graph_begin / _end / _launch), replayed with one call;
  * the operators also compose with torch.cuda.graph(): they launch on the current stream and
    allocate only through torch's allocator.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _capi as capi


class GraphedLayerNorm:
    """y = layer_norm(x) (optionally + GELU) on fixed buffers, replayed as one CUDA graph.

        g = GraphedLayerNorm(x_static, weight, bias, eps)      # records; does not execute
        x_static.copy_(new_x); y = g()                          # one graph launch
    `repeat` records the same call several times in one graph: what a stack of identical
    layers looks like to the launch path.
    """

    def __init__(self, x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                 eps: float = 1e-5, gelu: Optional[str] = None, repeat: int = 1):
        if not x.is_cuda or x.dim() != 2 or not x.is_contiguous():
            raise RuntimeError("GraphedLayerNorm needs a contiguous 2-D CUDA tensor")
        self.x, self.weight, self.bias = x, weight, bias
        self.y = torch.empty_like(x)
        self.mean = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        self.rstd = torch.empty_like(self.mean)
        self._g = capi.Graph()
        with torch.cuda.device(x.device):
            with self._g.record() as s:
                for _ in range(repeat):
                    if gelu is None:
                        capi.layernorm_forward(x, weight, bias, self.y, self.mean, self.rstd, eps, stream=s)
                    else:
                        act = capi.ACT_GELU_TANH if gelu == "tanh" else capi.ACT_GELU_ERF
                        capi.layernorm_gelu_forward(x, weight, bias, self.y, eps, act, stream=s)

    def __call__(self) -> torch.Tensor:
        self._g.launch()
        return self.y

    def close(self):
        self._g.close()


class GraphedLayerNormStep:
    """forward + backward (dx, dgamma, dbeta) on fixed buffers as one graph (two kernels where the
    backward reduces dgamma / dbeta in its own tail, three otherwise)."""

    def __init__(self, x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5):
        rows, cols = x.shape
        self.x, self.dy = x, dy
        self.y = torch.empty_like(x)
        self.dx = torch.empty_like(x)
        self.mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        self.rstd = torch.empty_like(self.mean)
        self.dweight = torch.empty_like(weight)
        self.dbias = torch.empty_like(bias)
        nbytes = capi.backward_workspace_bytes(rows, cols, x.dtype)
        self._ws = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=x.device)
        self._g = capi.Graph()
        with torch.cuda.device(x.device):
            with self._g.record() as s:
                capi.layernorm_forward(x, weight, bias, self.y, self.mean, self.rstd, eps, stream=s)
                capi.layernorm_backward(dy, x, self.mean, self.rstd, weight, self.dx, self.dweight, self.dbias,
                                        self._ws, stream=s)

    def __call__(self):
        self._g.launch()
        return self.y, self.dx, self.dweight, self.dbias

    def close(self):
        self._g.close()
