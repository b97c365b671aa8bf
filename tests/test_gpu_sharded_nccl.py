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
