"""Row-sharded LayerNorm forward + backward across the GPUs of one node.

Rows are independent, so a batch of `total_rows` rows is cut into contiguous, near-equal
shards, one per rank; gamma / beta are replicated.  The forward needs no communication.  The
backward needs exactly one exchange: the per-rank fp32 partial sums [dgamma | dbeta] (one
contiguous buffer of 2 * hidden floats, written by the column-reduction kernel with no
rounding) are summed with a single all-reduce, and only then rounded to the parameter dtype.
On GPUs the process group is NCCL (NVLink / NVSwitch); the reference has no multi-GPU code
at all.  Nothing here puts kernels of different ranks on one GPU or waits on a peer from
inside a kernel: the only cross-rank synchronization is the collective itself.

The local computation is injected (`backend`) so that the sharding / reduction logic can be
exercised on CPU ranks over gloo with a checker as the backend; the default backend is the
CUDA operator set and raises if the extension is missing.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, end) of rank's shard: ceil-split, later ranks may get fewer (or zero) rows."""
    if total_rows < 0 or world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad sharding request: rows={total_rows} world={world_size} rank={rank}")
    per = -(-total_rows // world_size)
    start = min(rank * per, total_rows)
    return start, min(start + per, total_rows)


class CudaBackend:
    """Local compute on the current CUDA device through the registered operators."""

    def __init__(self):
        from . import ops as _ops  # noqa: F401  (raises ImportError when the extension is missing)
        self._t = torch.ops.fused_layernorm

    def forward(self, x, gamma, beta, eps):
        return self._t.layernorm_fwd(x, gamma, beta, eps)

    def backward_f32(self, dy, x, mean, rstd, gamma):
        return self._t.layernorm_bwd_f32(dy, x, mean, rstd, gamma)

    def cast(self, f32, dtype):
        return self._t.cast_from_f32(f32, dtype)


class ShardedLayerNorm:
    """forward / backward of one rank's shard, plus the all-reduce of the parameter gradients.

        sln = ShardedLayerNorm(hidden, eps)            # after dist.init_process_group(...)
        y, saved = sln.forward(x_shard, gamma, beta)
        dx, dgamma, dbeta = sln.backward(dy_shard, saved, gamma)
    """

    def __init__(self, hidden: int, eps: float = 1e-5, group=None, backend=None, sm_reserve: Optional[int] = 2):
        self.hidden = int(hidden)
        self.eps = float(eps)
        self.group = group
        self.backend = backend if backend is not None else CudaBackend()
        # The persistent kernels fill every SM; a collective kernel that runs beside them (the
        # asynchronous all-reduce of the previous step) then delays some of their CTAs.  With
        # more than one rank the default CUDA backend leaves `sm_reserve` SMs free (a
        # process-wide setting of the library; None leaves it untouched).  8 GPUs, 16384 x 8192
        # bf16 per rank: 0.284 ms per step with 0 SMs free, 0.263 with 2.
        if backend is None and sm_reserve is not None and dist.is_available() and dist.is_initialized() \
                and dist.get_world_size(group) > 1:
            from . import _capi
            _capi.lib().fln_set_sm_reserve(int(sm_reserve))

    # -- checks that run on the host before anything is launched -------------------------
    def _check_shard(self, t: torch.Tensor, name: str):
        if t.dim() != 2 or t.shape[1] != self.hidden:
            raise ValueError(f"{name} must be [rows, {self.hidden}], got {tuple(t.shape)}")

    def validate(self, local_rows: int, total_rows: Optional[int] = None):
        """Collective sanity check (call it once, not per step): every rank uses the same
        hidden size and, when total_rows is given, the shard sizes are those of shard_bounds."""
        world = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        mine = torch.tensor([self.hidden, local_rows], dtype=torch.int64)
        if dist.get_backend(self.group) == "nccl":
            mine = mine.cuda()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=self.group)
        hs = [int(g[0]) for g in gathered]
        rows = [int(g[1]) for g in gathered]
        if len(set(hs)) != 1:
            raise RuntimeError(f"hidden size differs across ranks: {hs}")
        if total_rows is not None:
            want = [shard_bounds(total_rows, world, r) for r in range(world)]
            if rows != [b - a for a, b in want]:
                raise RuntimeError(f"shard sizes {rows} do not match an even split of {total_rows} rows over {world} ranks")
        return rows[rank]

    # -- the path ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor]):
        self._check_shard(x, "x")
        y, mean, rstd = self.backend.forward(x, gamma, beta, self.eps)
        return y, (x, mean, rstd)

    def backward(self, dy: torch.Tensor, saved, gamma: Optional[torch.Tensor], async_op: bool = False):
        """Returns (dx, dgamma, dbeta); dgamma / dbeta are the sums over ALL ranks' rows, in the
        dtype of x.  With async_op=True returns (dx, finish) where finish() waits for the
        all-reduce and returns (dgamma, dbeta), so the caller can overlap it with other work."""
        x, mean, rstd = saved
        self._check_shard(dy, "dy")
        if dy.shape != x.shape:
            raise ValueError(f"dy shape {tuple(dy.shape)} does not match x shape {tuple(x.shape)}")
        dx, dgb = self.backend.backward_f32(dy, x, mean, rstd, gamma)  # dgb: fp32 [2 * hidden], zeros for an empty shard
        work = dist.all_reduce(dgb, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

        def finish():
            work.wait()
            out = self.backend.cast(dgb, x.dtype)
            return out[: self.hidden], out[self.hidden:]

        if async_op:
            return dx, finish
        dgamma, dbeta = finish()
        return dx, dgamma, dbeta


class ShardedLayerNormStep:
    """The training step of one rank, preallocated: LayerNorm forward + backward over this rank's
    shard with the sums of the parameter gradients off the critical path.

        step = ShardedLayerNormStep(rows, hidden, torch.bfloat16)   # after init_process_group
        for batch in loader:
            y = step.forward(x, gamma, beta)           # current stream, no communication
            dx = step.backward(dy, gamma)              # current stream; the sums are queued
            ...
        dgamma, dbeta = step.finish()                  # joins the sums still in flight

    The backward launched on the caller's stream is stage 1 only (dx and the per-CTA partial sums
    of dgamma / dbeta): its kernel ends without a grid-wide barrier, so whatever the caller
    launches next starts while its last CTAs finish.  The column sum of the partial rows, the
    all-reduce of the fp32 [dgamma | dbeta] over the ranks (when there are several) and the
    rounding to the parameter dtype run on a side stream, behind an event that follows the
    backward; the caller's stream never waits for them (a training loop needs the parameter
    gradients at its optimizer step, not before), so they overlap the next forward.  Two sets of
    buffers alternate; before a set is written again the caller's stream waits for the event that
    marks its previous sums as finished, which by then lies a whole step in the past.
    Everything is launched through the C ABI on buffers allocated here once, so a step allocates
    nothing.  No kernel of this class waits on a peer; the only cross-rank synchronization is
    the collective.
    """

    def __init__(self, rows: int, hidden: int, dtype=torch.bfloat16, eps: float = 1e-5, group=None,
                 sm_reserve: Optional[int] = 2, device=None):
        from . import _capi as capi  # raises when the library has not been built: no fallback
        self._capi = capi
        self.rows, self.hidden, self.dtype, self.eps, self.group = int(rows), int(hidden), dtype, float(eps), group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        d = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = d
        if self.world > 1 and sm_reserve is not None:
            capi.lib().fln_set_sm_reserve(int(sm_reserve))  # see ShardedLayerNorm.__init__
        self.y = torch.empty(rows, hidden, dtype=dtype, device=d)
        self.dx = torch.empty(rows, hidden, dtype=dtype, device=d)
        self.mean = torch.empty(rows, dtype=torch.float32, device=d)
        self.rstd = torch.empty(rows, dtype=torch.float32, device=d)
        self.dgb = [torch.zeros(2 * hidden, dtype=torch.float32, device=d) for _ in range(2)]
        self.dparams = torch.zeros(2 * hidden, dtype=dtype, device=d)
        ws = capi.backward_workspace_bytes(rows, hidden, dtype)
        self.ws = [torch.empty(max(ws // 4, 1), dtype=torch.float32, device=d) for _ in range(2)]
        self.side = torch.cuda.Stream(d)
        self.ev_bwd = [torch.cuda.Event() for _ in range(2)]
        self.ev_red = [torch.cuda.Event() for _ in range(2)]
        self.steps = 0
        self._x = None
        # kernels of this library per step: forward, backward stage 1, the column sum of the
        # partial rows (which also rounds when there is one rank), and with more than one rank
        # the rounding of the all-reduced sums
        self.launches_per_step = 3 + (1 if self.world > 1 else 0)

    def forward(self, x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor]) -> torch.Tensor:
        if x.shape != (self.rows, self.hidden) or x.dtype != self.dtype:
            raise ValueError(f"x must be [{self.rows}, {self.hidden}] {self.dtype}, got {tuple(x.shape)} {x.dtype}")
        if self.rows:
            self._capi.layernorm_forward(x, gamma, beta, self.y, self.mean, self.rstd, self.eps)
        self._x = x
        return self.y

    def backward(self, dy: torch.Tensor, gamma: Optional[torch.Tensor]) -> torch.Tensor:
        capi = self._capi
        if self._x is None:
            raise RuntimeError("backward() before forward()")
        if dy.shape != self._x.shape or dy.dtype != self.dtype:
            raise ValueError(f"dy must match x: {tuple(self._x.shape)} {self.dtype}")
        k = self.steps & 1
        buf = self.dgb[k]
        main = torch.cuda.current_stream(self.device)
        if self.steps >= 2:
            main.wait_event(self.ev_red[k])  # buffer set k is free again
        self.steps += 1
        partial = None
        if self.rows:
            partial = capi.norm_backward_partial(capi.LAYERNORM, dy, self._x, self.mean, self.rstd, gamma, None,
                                                 self.dx, self.ws[k])
        self.ev_bwd[k].record(main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(self.ev_bwd[k])
            if partial is not None and partial.shape[0] > 0:
                capi.sum_rows_f32(partial, buf, self.dparams if self.world == 1 else None, stream=self.side)
            else:
                buf.zero_()  # an empty shard contributes zeros
                if self.world == 1:
                    self.dparams.zero_()
            if self.world > 1:
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
                capi.cast_from_f32(buf, self.dparams, stream=self.side)
            self.ev_red[k].record(self.side)
        return self.dx

    def finish(self):
        """Makes the current stream wait for the sums still in flight and returns (dgamma,
        dbeta) of the last step, summed over all ranks, in the parameter dtype."""
        torch.cuda.current_stream(self.device).wait_stream(self.side)
        return self.dparams[: self.hidden], self.dparams[self.hidden:]

    def last_sums_f32(self) -> torch.Tensor:
        """The unrounded fp32 [dgamma | dbeta] of the last step (after finish(): summed over all
        ranks)."""
        return self.dgb[(self.steps - 1) & 1]
