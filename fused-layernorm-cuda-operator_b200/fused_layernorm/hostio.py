"""LayerNorm forward + backward for callers whose tensors live in host memory.

The batch is cut into row chunks; chunk i+1 is copied to the device while chunk i is being
normalized and the results of chunk i-1 travel back, on three CUDA streams.  Rows are
independent, so only dgamma / dbeta need a final step: every chunk leaves its unrounded fp32
[dgamma | dbeta] in its own slot and the slots are added at the end.

This is the path bench.py times as `e2e`: pinned host buffers in, pinned host buffers out,
all copies inside the timed region.
"""
from __future__ import annotations

import torch

from . import _capi as capi


class HostLayerNormFwdBwd:
    def __init__(self, rows: int, cols: int, dtype=torch.bfloat16, chunk_rows: int = 2048, device=None):
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.chunk_rows = min(chunk_rows, rows)
        self.bounds = [(r, min(r + self.chunk_rows, rows)) for r in range(0, rows, self.chunk_rows)]
        n = len(self.bounds)
        d = self.device
        self.x = torch.empty(rows, cols, dtype=dtype, device=d)
        self.dy = torch.empty_like(self.x)
        self.y = torch.empty_like(self.x)
        self.dx = torch.empty_like(self.x)
        self.mean = torch.empty(rows, dtype=torch.float32, device=d)
        self.rstd = torch.empty(rows, dtype=torch.float32, device=d)
        self.slots = torch.zeros(n, 2 * cols, dtype=torch.float32, device=d)
        self.dgb = torch.empty(2 * cols, dtype=torch.float32, device=d)
        self.dparams = torch.empty(2 * cols, dtype=dtype, device=d)
        # the last chunk may be shorter and planned differently: size for the largest request
        ws = max(capi.backward_workspace_bytes(b - a, cols, dtype) for a, b in self.bounds)
        self.ws = torch.empty(max(ws // 4, 1), dtype=torch.float32, device=d)
        self.s_in = torch.cuda.Stream(d)
        self.s_cmp = torch.cuda.Stream(d)
        self.s_out = torch.cuda.Stream(d)
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(n)]
        # forward + backward per chunk (the backward reduces its partial sums in its own tail at
        # these sizes; where it cannot, it adds a launch), one sum of the chunks' slots with the cast
        self.launches_per_call = 2 * n + 1

    @property
    def h2d_bytes(self) -> int:
        return 2 * self.rows * self.cols * self.x.element_size()

    @property
    def d2h_bytes(self) -> int:
        return 2 * self.rows * self.cols * self.x.element_size() + 2 * self.cols * self.x.element_size()

    def __call__(self, x_host, dy_host, gamma, beta, y_host, dx_host, dparams_host, eps: float = 1e-5):
        """x_host, dy_host: pinned [rows, cols]; gamma, beta: device [cols];
        y_host, dx_host: pinned [rows, cols]; dparams_host: pinned [2*cols] = [dgamma | dbeta].
        Returns after enqueueing; the caller synchronizes (or waits on the current stream,
        which is made to wait for all three internal streams)."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        for i, (a, b) in enumerate(self.bounds):
            with torch.cuda.stream(self.s_in):
                self.x[a:b].copy_(x_host[a:b], non_blocking=True)
                self.dy[a:b].copy_(dy_host[a:b], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[i])
                capi.layernorm_forward(self.x[a:b], gamma, beta, self.y[a:b], self.mean[a:b], self.rstd[a:b],
                                       eps, stream=self.s_cmp)
                capi.norm_backward(capi.LAYERNORM, self.dy[a:b], self.x[a:b], self.mean[a:b], self.rstd[a:b],
                                   gamma, None, self.dx[a:b], None, None, self.slots[i], self.ws,
                                   stream=self.s_cmp)
                self.ev_cmp[i].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[i])
                y_host[a:b].copy_(self.y[a:b], non_blocking=True)
                dx_host[a:b].copy_(self.dx[a:b], non_blocking=True)
        with torch.cuda.stream(self.s_cmp):
            capi.sum_rows_f32(self.slots, self.dgb, self.dparams, stream=self.s_cmp)
        self.s_out.wait_stream(self.s_cmp)
        with torch.cuda.stream(self.s_out):
            dparams_host.copy_(self.dparams, non_blocking=True)
        cur.wait_stream(self.s_out)
