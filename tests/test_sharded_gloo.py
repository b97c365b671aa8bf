"""The N > 1 path on CPU: two gloo ranks run the row-sharding + all-reduce logic of
fused_layernorm.sharded with the CPU checker injected as the local compute, and the result is
compared with the checker run once over the whole batch.  Also: uneven and empty shards, and
host-side failures (shape mismatch across ranks, bad shard shapes) raised before any launch."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


class OracleBackend:
    """Local compute through the CPU checker (test infrastructure, never the product path)."""

    def forward(self, x, gamma, beta, eps):
        from oracle import oracle as O
        r = O.norm_forward(x, gamma, beta, None, "layernorm", eps)
        return r["y"], r["mean"], r["rstd"]

    def backward_f32(self, dy, x, mean, rstd, gamma):
        from oracle import oracle as O
        if x.shape[0] == 0:
            return torch.empty_like(x), torch.zeros(2 * x.shape[1], dtype=torch.float32)
        r = O.norm_backward(dy, x, mean, rstd, gamma)
        return r["dx"], torch.cat([r["dgamma64"], r["dbeta64"]]).float()

    def cast(self, f32, dtype):
        return f32.to(dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total_rows, hidden, mode, out_dir):
    for p in (str(ROOT), str(ROOT / "fused-layernorm-cuda-operator_b200"), str(ROOT / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fused_layernorm.sharded import ShardedLayerNorm, shard_bounds
        g = torch.Generator().manual_seed(20245)
        x = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
        dy = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        beta = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        a, b = shard_bounds(total_rows, world, rank)
        sln = ShardedLayerNorm(hidden if not (mode == "hidden_mismatch" and rank == 1) else hidden + 8, 1e-5,
                               backend=OracleBackend())
        if mode == "hidden_mismatch":
            try:
                sln.validate(b - a, total_rows)
                result = "no error"
            except RuntimeError as e:
                result = str(e)
            torch.save(result, f"{out_dir}/r{rank}.pt")
            return
        if mode == "bad_shard":
            try:
                sln.forward(x[a:b, : hidden - 1], gamma, beta)
                result = "no error"
            except ValueError as e:
                result = str(e)
            torch.save(result, f"{out_dir}/r{rank}.pt")
            return
        assert sln.validate(b - a, total_rows) == b - a
        y, saved = sln.forward(x[a:b].contiguous(), gamma, beta)
        if mode == "async":
            dx, finish = sln.backward(dy[a:b].contiguous(), saved, gamma, async_op=True)
            dgamma, dbeta = finish()
        else:
            dx, dgamma, dbeta = sln.backward(dy[a:b].contiguous(), saved, gamma)
        torch.save({"y": y, "dx": dx, "dgamma": dgamma, "dbeta": dbeta, "bounds": (a, b)}, f"{out_dir}/r{rank}.pt")
    finally:
        dist.destroy_process_group()


def _run(world, total_rows, hidden, mode, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, total_rows, hidden, mode, str(tmp_path)), nprocs=world, join=True)
    return [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]


@pytest.mark.parametrize("total_rows,mode", [(64, "sync"), (37, "sync"), (1, "sync"), (64, "async")])
def test_two_ranks_match_single_process(tmp_path, total_rows, mode):
    from oracle import oracle as O
    hidden = 256
    outs = _run(2, total_rows, hidden, mode, tmp_path)
    g = torch.Generator().manual_seed(20245)
    x = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
    dy = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    f = O.norm_forward(x, gamma, beta)
    b = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
    assert sum(o["bounds"][1] - o["bounds"][0] for o in outs) == total_rows
    y = torch.cat([o["y"] for o in outs])
    dx = torch.cat([o["dx"] for o in outs])
    assert torch.equal(y.view(torch.int16), f["y"].view(torch.int16))
    assert torch.equal(dx.view(torch.int16), b["dx"].view(torch.int16))
    for o in outs:  # every rank holds the global sums
        assert int(O.mismatch_16(o["dgamma"], b["dgamma"]).sum()) == 0
        assert int(O.mismatch_16(o["dbeta"], b["dbeta"]).sum()) == 0
    assert torch.equal(outs[0]["dgamma"].view(torch.int16), outs[1]["dgamma"].view(torch.int16))


def test_hidden_size_mismatch_is_reported_on_every_rank(tmp_path):
    outs = _run(2, 16, 64, "hidden_mismatch", tmp_path)
    assert all("hidden size differs across ranks" in o for o in outs)


def test_bad_shard_shape_raises_before_any_compute(tmp_path):
    outs = _run(2, 16, 64, "bad_shard", tmp_path)
    assert all("must be [rows, 64]" in o for o in outs)
