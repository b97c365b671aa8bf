"""The give-up paths of the pipelined kernels, exercised without faulting or hanging the GPU.

Every wait inside these kernels is bounded by elapsed time.  The library has two test hooks,
both host-settable words the kernels read: one makes CTA 0 arm its first stage without issuing
the copy (so the wait for that stage runs out), one makes the backward's grid barrier expect a
CTA more than the grid has (so every CTA's wait runs out).  With the limit lowered to a few
milliseconds each launch below returns on its own through its ordinary give-up path; the tests
check the status word, that the launch left the barrier word and the forward's tile counter
ready for the next launch, and that the next ordinary call -- eager and as a replay of a CUDA
graph recorded earlier -- is correct again.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as U
    from fused_layernorm import _capi as capi
    from oracle import oracle as O

BF16 = torch.bfloat16
ROWS, COLS = 4096, 8192  # pipelined in both directions, fused column reduce
LIMIT_NS = 3_000_000


@pytest.fixture
def hooks():
    L = capi.lib()
    assert L.fln_device_status() == 0
    assert L.fln_set_wait_limit_ns(LIMIT_NS) == 0
    yield L
    L.fln_set_test_fault(0)
    L.fln_set_wait_limit_ns(0)
    torch.cuda.synchronize()
    L.fln_device_status()


def _problem(seed=5):
    x, gamma, beta, dy, _ = U.make_inputs(seed, ROWS, COLS, BF16)
    f = O.norm_forward(x, gamma, beta)
    return x, gamma, beta, dy, f


def _backward_buffers():
    return dict(dx=torch.empty(ROWS, COLS, dtype=BF16, device="cuda"),
                dgb=torch.empty(2 * COLS, device="cuda"),
                ws=torch.empty(capi.backward_workspace_bytes(ROWS, COLS, BF16) // 4, device="cuda"))


def _check_backward(b, dy, x, f, gamma):
    want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
    U.assert_out_close(b["dx"].cpu(), want["dx"], BF16)
    U.assert_param_grads_close(b["dgb"].cpu(), torch.cat([want["dgamma64"], want["dbeta64"]]),
                               want["abs64"].reshape(-1), ROWS)


def test_describe_says_both_directions_are_pipelined():
    assert capi.describe_launch(False, ROWS, COLS, BF16)["pipelined"] == 1
    assert capi.describe_launch(True, ROWS, COLS, BF16)["pipelined"] == 1


def test_grid_barrier_gives_up_and_the_next_calls_are_correct(hooks):
    x, gamma, beta, dy, f = _problem()
    d = [t.cuda() for t in (dy, x, f["mean"], f["rstd"], gamma)]
    b = _backward_buffers()
    run = lambda stream=None: capi.norm_backward(capi.LAYERNORM, d[0], d[1], d[2], d[3], d[4], None, b["dx"], None,
                                                 None, b["dgb"], b["ws"], stream=stream)
    # a graph recorded while everything is in order: its launch token is baked in
    g = capi.Graph()
    with g.record() as stream:
        run(stream)
    g.launch()
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 0
    _check_backward(b, dy, x, f, gamma)

    hooks.fln_set_test_fault(2)
    b["dgb"].fill_(7.0)
    run()
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 2          # read and cleared
    assert hooks.fln_device_status() == 0
    assert float(b["dgb"].min()) == 7.0            # no CTA summed the partial rows
    g.launch()                                      # the same give-up under the graph's token
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 2

    hooks.fln_set_test_fault(0)
    b["dx"].zero_()
    g.launch()                                      # same token again: the word must have been left clean
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 0
    _check_backward(b, dy, x, f, gamma)
    b["dx"].zero_()
    b["dgb"].fill_(7.0)
    run()
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 0
    _check_backward(b, dy, x, f, gamma)


def test_backward_stage_wait_gives_up_and_the_next_call_is_correct(hooks):
    x, gamma, beta, dy, f = _problem(6)
    d = [t.cuda() for t in (dy, x, f["mean"], f["rstd"], gamma)]
    b = _backward_buffers()
    run = lambda: capi.norm_backward(capi.LAYERNORM, d[0], d[1], d[2], d[3], d[4], None, b["dx"], None, None,
                                     b["dgb"], b["ws"])
    hooks.fln_set_test_fault(1)
    run()
    torch.cuda.synchronize()
    status = hooks.fln_device_status()
    assert status & 1                               # CTA 0 gave up on its first stage ...
    assert status & ~3 == 0                         # ... and the others, at most, on the barrier
    hooks.fln_set_test_fault(0)
    b["dx"].zero_()
    run()
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 0
    _check_backward(b, dy, x, f, gamma)


def test_forward_stage_wait_gives_up_and_the_next_call_is_correct(hooks):
    x, gamma, beta, dy, f = _problem(7)
    xd, gd, bd = x.cuda(), gamma.cuda(), beta.cuda()
    y = torch.zeros(ROWS, COLS, dtype=BF16, device="cuda")
    mean = torch.empty(ROWS, device="cuda")
    rstd = torch.empty(ROWS, device="cuda")
    run = lambda: capi.layernorm_forward(xd, gd, bd, y, mean, rstd, 1e-5)
    hooks.fln_set_test_fault(1)
    run()
    torch.cuda.synchronize()
    assert hooks.fln_device_status() == 1
    hooks.fln_set_test_fault(0)
    # The launch that gave up must have handed its pair of tile counters back at zero.  Launches
    # take the pairs of a ring of 1024 in turn, so go once around the ring and a little further.
    for lap in range(2):
        y.zero_()
        for _ in range(520):
            run()
        torch.cuda.synchronize()
        assert hooks.fln_device_status() == 0
        U.assert_out_close(y.cpu(), f["y"], BF16)
        torch.testing.assert_close(mean.cpu(), f["mean"], rtol=1e-5, atol=1e-5)


def test_cluster_pair_gives_up_together_and_the_next_call_is_correct(hooks):
    """A row shared by the two CTAs of a cluster: CTA 0 never gets its first copy, so its wait
    runs out; its partner then waits in vain for CTA 0's row sums and gives up too (that wait is
    bounded like the others).  Both leave through the ordinary exit, the status word says 1,
    and the next call is correct."""
    rows, cols = 600, 16384
    F32 = torch.float32
    hooks.fln_set_path_override(2)
    try:
        d = capi.describe_launch(True, rows, cols, F32)
        assert d["pipelined"] == 1 and 2 * d["vecs_per_thread"] * (d["vector_bytes"] // 4) * 512 == cols
        x, gamma, beta, dy, _ = U.make_inputs(11, rows, cols, F32)
        f = O.norm_forward(x, gamma, beta)
        dev = [t.cuda() for t in (dy, x, f["mean"], f["rstd"], gamma)]
        dx = torch.zeros(rows, cols, device="cuda")
        dgb = torch.empty(2 * cols, device="cuda")
        ws = torch.empty(capi.backward_workspace_bytes(rows, cols, F32) // 4, device="cuda")
        run = lambda: capi.norm_backward(capi.LAYERNORM, dev[0], dev[1], dev[2], dev[3], dev[4], None, dx, None, None,
                                         dgb, ws)
        hooks.fln_set_test_fault(1)
        run()
        torch.cuda.synchronize()
        assert hooks.fln_device_status() == 1
        hooks.fln_set_test_fault(0)
        dx.zero_()
        run()
        torch.cuda.synchronize()
        assert hooks.fln_device_status() == 0
        want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
        torch.testing.assert_close(dx.cpu(), want["dx32"], rtol=1e-5, atol=1e-5)
        U.assert_param_grads_close(dgb.cpu(), torch.cat([want["dgamma64"], want["dbeta64"]]), want["abs64"].reshape(-1), rows)
    finally:
        hooks.fln_set_path_override(0)


def test_two_pass_backward_gives_up_and_the_next_call_is_correct(hooks):
    """16-bit rows of 16384 columns (one CTA per row, two passes over the staged row): CTA 0 never
    gets its first copy, its wait runs out, the launch returns with status 1, and the next call
    is correct."""
    rows, cols = 600, 16384
    hooks.fln_set_path_override(2)
    try:
        d = capi.describe_launch(True, rows, cols, BF16)
        assert d["pipelined"] == 1 and d["vecs_per_thread"] == 4 and d["threads_per_row"] == 512 and d["stages"] == 2
        x, gamma, beta, dy, _ = U.make_inputs(12, rows, cols, BF16)
        f = O.norm_forward(x, gamma, beta)
        dev = [t.cuda() for t in (dy, x, f["mean"], f["rstd"], gamma)]
        dx = torch.zeros(rows, cols, dtype=BF16, device="cuda")
        dgb = torch.empty(2 * cols, device="cuda")
        ws = torch.empty(capi.backward_workspace_bytes(rows, cols, BF16) // 4, device="cuda")
        run = lambda: capi.norm_backward(capi.LAYERNORM, dev[0], dev[1], dev[2], dev[3], dev[4], None, dx, None, None,
                                         dgb, ws)
        hooks.fln_set_test_fault(1)
        run()
        torch.cuda.synchronize()
        assert hooks.fln_device_status() == 1
        hooks.fln_set_test_fault(0)
        dx.zero_()
        run()
        torch.cuda.synchronize()
        assert hooks.fln_device_status() == 0
        want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
        U.assert_out_close(dx.cpu(), want["dx"], BF16)
        U.assert_param_grads_close(dgb.cpu(), torch.cat([want["dgamma64"], want["dbeta64"]]), want["abs64"].reshape(-1), rows)
    finally:
        hooks.fln_set_path_override(0)
