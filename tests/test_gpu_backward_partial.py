"""Stage 1 of the backward on its own (fln_norm_backward_partial) and the deferred column sum
(fln_sum_rows_f32), and the preallocated training step built on them
(fused_layernorm.sharded.ShardedLayerNormStep with one rank): dx and the parameter gradients
against the CPU checker, over several steps with different data so that the alternating buffer
sets are exercised."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as U
    from fused_layernorm import _capi as capi
    from oracle import oracle as O

BF16, F32 = torch.bfloat16, torch.float32


@pytest.mark.parametrize("rows,cols,dtype", [(4096, 8192, BF16), (4096, 4096, BF16), (2048, 5120, BF16),
                                             (4096, 2048, F32), (33, 1023, BF16), (64, 768, F32), (3000, 1600, BF16)])
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
def test_partial_backward_plus_row_sum_matches_checker(rows, cols, dtype, kind):
    x, gamma, beta, dy, _ = U.make_inputs(31, rows, cols, dtype)
    f = O.norm_forward(x, gamma, beta if kind == "layernorm" else None, kind=kind)
    want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma, kind=kind)
    nr = 2 if kind == "layernorm" else 1
    d = lambda t: None if t is None else t.cuda()
    dx = U.Guarded((rows, cols), dtype)
    ws = U.Guarded((max(capi.backward_workspace_bytes(rows, cols, dtype) // 4, 1),), F32)
    part = capi.norm_backward_partial(U.KINDS[kind], d(dy), d(x), d(f["mean"]), d(f["rstd"]), d(gamma), None, dx.t, ws.t)
    assert part.shape[1] == nr * cols and part.shape[0] >= 1
    sums = U.Guarded((nr * cols,), F32)
    cast = U.Guarded((nr * cols,), dtype)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    capi.sum_rows_f32(part, sums.t, cast.t, stream=side)  # on another stream, as a training step would
    torch.cuda.synchronize()
    ws.check()
    if dtype == F32:
        torch.testing.assert_close(dx.check().cpu(), want["dx32"], rtol=1e-5, atol=1e-5)
    else:
        U.assert_out_close(dx.check().cpu(), want["dx"], dtype)
    got = sums.check().cpu()
    U.assert_param_grads_close(got[:cols], want["dgamma64"], want["abs64"][0], rows)
    if kind == "layernorm":
        U.assert_param_grads_close(got[cols:], want["dbeta64"], want["abs64"][1], rows)
    assert torch.equal(cast.check().cpu(), got.to(dtype))  # the rounded copy is the rounding of the fp32 sums
    assert capi.lib().fln_device_status() == 0


def test_partial_backward_agrees_bitwise_with_the_two_kernel_backward():
    """Same stage-1 kernel, same fixed-order column sum: identical bits as the regular entry
    point when that is told to reduce with a second kernel."""
    rows, cols = 4096, 8192
    x, gamma, beta, dy, _ = U.make_inputs(32, rows, cols, BF16)
    f = O.norm_forward(x, gamma, beta)
    L = capi.lib()
    L.fln_set_path_override(3)
    try:
        ref = U.run_backward(dy, x, f["mean"], f["rstd"], gamma)
    finally:
        L.fln_set_path_override(0)
    d = lambda t: t.cuda()
    dx = torch.empty(rows, cols, dtype=BF16, device="cuda")
    ws = torch.empty(capi.backward_workspace_bytes(rows, cols, BF16) // 4, device="cuda")
    part = capi.norm_backward_partial(capi.LAYERNORM, d(dy), d(x), d(f["mean"]), d(f["rstd"]), d(gamma), None, dx, ws)
    sums = torch.empty(2 * cols, device="cuda")
    capi.sum_rows_f32(part, sums, None)
    torch.cuda.synchronize()
    assert torch.equal(dx.cpu(), ref["dx"])
    assert torch.equal(sums.cpu(), ref["dgb_f32"])


def test_empty_batch_reports_no_partial_rows():
    ws = torch.empty(1024, device="cuda")
    x = torch.empty(0, 256, dtype=BF16, device="cuda")
    st = torch.empty(0, device="cuda")
    part = capi.norm_backward_partial(capi.LAYERNORM, x, x, st, st, None, None, x, ws)
    assert part.shape == (0, 512)


@pytest.mark.parametrize("rows,cols", [(4096, 8192), (1000, 1024), (0, 512)])
def test_single_rank_training_step_over_several_steps(rows, cols):
    from fused_layernorm.sharded import ShardedLayerNormStep
    step = ShardedLayerNormStep(rows, cols, BF16)
    assert step.world == 1
    gamma = beta = None
    for seed in (1, 2, 3):  # three steps: both buffer sets get reused
        x, gamma, beta, dy, _ = U.make_inputs(seed, rows, cols, BF16)
        xd, dyd, gd, bd = x.cuda(), dy.cuda(), gamma.cuda(), beta.cuda()
        y = step.forward(xd, gd, bd)
        dx = step.backward(dyd, gd)
        dgamma, dbeta = step.finish()
        torch.cuda.synchronize()
        if rows == 0:
            assert float(dgamma.float().abs().max()) == 0.0 and float(dbeta.float().abs().max()) == 0.0
            continue
        f = O.norm_forward(x, gamma, beta)
        want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
        U.assert_out_close(y.cpu(), f["y"], BF16)
        U.assert_out_close(dx.cpu(), want["dx"], BF16)
        sums = step.last_sums_f32().cpu()
        U.assert_param_grads_close(sums[:cols], want["dgamma64"], want["abs64"][0], rows)
        U.assert_param_grads_close(sums[cols:], want["dbeta64"], want["abs64"][1], rows)
        assert torch.equal(torch.cat([dgamma, dbeta]).cpu(), sums.to(BF16))
    assert capi.lib().fln_device_status() == 0
