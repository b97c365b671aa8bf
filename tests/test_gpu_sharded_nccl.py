"""Row-sharded LayerNorm forward + backward on two GPUs over NCCL (one process per GPU), against
the CPU checker run once over the whole batch.  Skipped on machines with fewer than two GPUs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total_rows, hidden, out_dir):
    for p in (str(ROOT), str(ROOT / "fused-layernorm-cuda-operator_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from fused_layernorm.sharded import ShardedLayerNorm, shard_bounds
        g = torch.Generator().manual_seed(20245)
        x = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
        dy = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).cuda()
        beta = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).cuda()
        a, b = shard_bounds(total_rows, world, rank)
        sln = ShardedLayerNorm(hidden, 1e-5)
        sln.validate(b - a, total_rows)
        y, saved = sln.forward(x[a:b].cuda(), gamma, beta)
        dx, dgamma, dbeta = sln.backward(dy[a:b].cuda(), saved, gamma)
        torch.cuda.synchronize()
        torch.save({"y": y.cpu(), "dx": dx.cpu(), "dgamma": dgamma.cpu(), "dbeta": dbeta.cpu()}, f"{out_dir}/r{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total_rows,hidden", [(4096 + 7, 2048), (3, 1024)])
def test_two_gpu_sharded_step_matches_checker(tmp_path, total_rows, hidden):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import oracle as O
    mp.spawn(_worker, args=(2, _free_port(), total_rows, hidden, str(tmp_path)), nprocs=2, join=True)
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(2)]
    g = torch.Generator().manual_seed(20245)
    x = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
    dy = torch.randn(total_rows, hidden, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    f = O.norm_forward(x, gamma, beta)
    b = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
    assert int(O.mismatch_16(torch.cat([o["y"] for o in outs]), f["y"]).sum()) == 0
    assert int(O.mismatch_16(torch.cat([o["dx"] for o in outs]), b["dx"]).sum()) == 0
    for o in outs:
        assert int(O.mismatch_16(o["dgamma"], b["dgamma"], abs_floor=2e-2).sum()) == 0
        assert int(O.mismatch_16(o["dbeta"], b["dbeta"], abs_floor=2e-2).sum()) == 0
    assert torch.equal(outs[0]["dgamma"].view(torch.int16), outs[1]["dgamma"].view(torch.int16))


def _step_worker(rank, world, port, rows_per_rank, hidden, out_dir):
    for p in (str(ROOT), str(ROOT / "fused-layernorm-cuda-operator_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from fused_layernorm.sharded import ShardedLayerNormStep
        step = ShardedLayerNormStep(rows_per_rank, hidden, torch.bfloat16)
        out = []
        for it in range(3):  # three steps: both buffer sets of the step object get reused
            g = torch.Generator().manual_seed(500 + 10 * it + rank)
            x = torch.randn(rows_per_rank, hidden, generator=g).to(torch.bfloat16)
            dy = torch.randn(rows_per_rank, hidden, generator=g).to(torch.bfloat16)
            gp = torch.Generator().manual_seed(77)
            gamma = (1 + 0.1 * torch.randn(hidden, generator=gp)).to(torch.bfloat16).cuda()
            beta = (0.1 * torch.randn(hidden, generator=gp)).to(torch.bfloat16).cuda()
            y = step.forward(x.cuda(), gamma, beta)
            dx = step.backward(dy.cuda(), gamma)
            dgamma, dbeta = step.finish()
            torch.cuda.synchronize()
            out.append({"y": y.cpu(), "dx": dx.cpu(), "dgamma": dgamma.cpu(), "dbeta": dbeta.cpu(),
                        "sums": step.last_sums_f32().cpu()})
        torch.save(out, f"{out_dir}/s{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_two_gpu_training_step_object_matches_checker(tmp_path):
    """fused_layernorm.sharded.ShardedLayerNormStep on two ranks: stage-1 backward on the main
    stream, column sum + all-reduce + rounding on the side stream, over three steps."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import oracle as O
    import gpu_util as U
    rows, hidden = 2048, 4096
    mp.spawn(_step_worker, args=(2, _free_port(), rows, hidden, str(tmp_path)), nprocs=2, join=True)
    outs = [torch.load(tmp_path / f"s{r}.pt") for r in range(2)]
    gp = torch.Generator().manual_seed(77)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=gp)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(hidden, generator=gp)).to(torch.bfloat16)
    for it in range(3):
        dg64 = torch.zeros(hidden, dtype=torch.float64)
        db64 = torch.zeros(hidden, dtype=torch.float64)
        abs64 = torch.zeros(2, hidden, dtype=torch.float64)
        for rank in range(2):
            g = torch.Generator().manual_seed(500 + 10 * it + rank)
            x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
            dy = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
            f = O.norm_forward(x, gamma, beta)
            b = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
            assert int(O.mismatch_16(outs[rank][it]["y"], f["y"]).sum()) == 0
            assert int(O.mismatch_16(outs[rank][it]["dx"], b["dx"]).sum()) == 0
            dg64 += b["dgamma64"]
            db64 += b["dbeta64"]
            abs64 += b["abs64"]
        for rank in range(2):
            sums = outs[rank][it]["sums"]
            U.assert_param_grads_close(sums[:hidden], dg64, abs64[0], 2 * rows)
            U.assert_param_grads_close(sums[hidden:], db64, abs64[1], 2 * rows)
            assert torch.equal(torch.cat([outs[rank][it]["dgamma"], outs[rank][it]["dbeta"]]), sums.to(torch.bfloat16))
        assert torch.equal(outs[0][it]["sums"], outs[1][it]["sums"])  # every rank holds the same sums
