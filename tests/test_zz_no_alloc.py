"""The allocation-free LayerNorm backward (fln_layernorm_backward_static), called through the C ABI.

Some hosts may not allocate device memory while they run -- a server with a fixed memory plan,
a loop that cannot take the device-wide synchronization of cudaMalloc -- so this entry point
keeps its scratch in an array built into the library instead of asking the caller for one.
Checked here: on two calls in a row (different inputs, so stale scratch contents would show) it
returns what the regular entry point returns, within the tolerance the other tests use (fp32
1e-5 abs/rel, bf16 one unit in the last place; in fact the two run the same kernels and agree
bit for bit); it refuses problems larger than its array; and it does not touch torch's
allocator.  The file name keeps it last in collection order, and it passes both alone in a
fresh process and after the rest of the suite.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as U
    from fused_layernorm import _capi as capi
    from oracle import oracle as O

F32, BF16 = torch.float32, torch.bfloat16


def _both(dy, x, mean, rstd, gamma, dtype):
    rows, cols = x.shape
    d = lambda t: t.cuda()
    dyd, xd, md, rd, gd = d(dy), d(x), d(mean), d(rstd), d(gamma)
    ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, dtype) // 4, 1), device="cuda")
    ref = [torch.empty(rows, cols, dtype=dtype, device="cuda"), torch.empty(cols, dtype=dtype, device="cuda"),
           torch.empty(cols, dtype=dtype, device="cuda")]
    capi.layernorm_backward(dyd, xd, md, rd, gd, ref[0], ref[1], ref[2], ws)
    got = [U.Guarded((rows, cols), dtype), U.Guarded((cols,), dtype), U.Guarded((cols,), dtype)]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    capi.layernorm_backward_static(dyd, xd, md, rd, gd, got[0].t, got[1].t, got[2].t)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return [r.cpu() for r in ref], [g.check().cpu() for g in got]


@pytest.mark.parametrize("dtype,shape", [(F32, (96, 1024)), (BF16, (4096, 2048)), (BF16, (33, 1023))])
def test_static_scratch_backward_matches_regular_entry_point_twice_in_a_row(dtype, shape):
    rows, cols = shape
    for call, seed in enumerate((101, 202)):  # second call: new data over the first call's leftovers
        x, gamma, beta, dy, _ = U.make_inputs(seed, rows, cols, dtype, x_scale=1.0 + call)
        f = O.norm_forward(x, gamma, beta)
        ref, got = _both(dy, x, f["mean"], f["rstd"], gamma, dtype)
        for r, g in zip(ref, got):
            U.assert_out_close(g, r, dtype)
            assert torch.equal(g, r)
        # and both agree with the checker
        want = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
        if dtype == F32:
            torch.testing.assert_close(got[0], want["dx32"], rtol=1e-5, atol=1e-5)
        else:
            U.assert_out_close(got[0], want["dx"], dtype)


def test_static_scratch_after_a_larger_plan_left_data_under_the_barrier_word():
    """The fused column reduce keeps its 8-byte barrier word right behind the partial rows, so the
    word's offset depends on the plan.  A 20-columns-per-thread plan (5120 columns) writes partial
    sums over the place where the 16-columns-per-thread plan (2048 columns) keeps its word; the
    second call must cope with floats there (the word needs no zeroing) and match the regular
    entry point bit for bit."""
    big = capi.backward_workspace_bytes(4096, 5120, BF16)
    small = capi.backward_workspace_bytes(4096, 2048, BF16)
    assert small < big <= capi.STATIC_SCRATCH_BYTES
    for rows, cols, seed in ((4096, 5120, 11), (4096, 2048, 12)):
        x, gamma, beta, dy, _ = U.make_inputs(seed, rows, cols, BF16)
        f = O.norm_forward(x, gamma, beta)
        ref, got = _both(dy, x, f["mean"], f["rstd"], gamma, BF16)
        for r, g in zip(ref, got):
            assert torch.equal(g, r)
    assert capi.lib().fln_device_status() == 0


def test_static_scratch_refuses_problems_beyond_its_capacity():
    """No plan of the launcher needs more than 19.4 MB on a B200 (checked over a grid of shapes),
    so the refusal is exercised by lowering the accepted size with the library's own hook: the
    call must return the static-scratch error and launch nothing."""
    L = capi.lib()
    worst = 0
    for dtype in (BF16, F32):
        for cols in (256, 512, 1024, 1280, 2048, 4096, 5120, 6144, 8192, 12288, 16384, 32768):
            for rows in (64, 600, 4096, 16384, 65536, 131072):
                for override in (0, 1, 2):
                    L.fln_set_path_override(override)
                    worst = max(worst, capi.backward_workspace_bytes(rows, cols, dtype))
    L.fln_set_path_override(0)
    assert worst <= capi.STATIC_SCRATCH_BYTES, worst
    rows, cols = 4096, 8192
    need = capi.backward_workspace_bytes(rows, cols, BF16)
    x = torch.zeros(rows, cols, dtype=BF16, device="cuda")
    st = torch.zeros(rows, device="cuda")
    dg = torch.full((cols,), 3.0, dtype=BF16, device="cuda")
    L.fln_set_static_scratch_limit(need - 1)
    try:
        with pytest.raises(RuntimeError, match="built-in static array"):
            capi.layernorm_backward_static(x, x, st, st, None, x, dg, None)
        torch.cuda.synchronize()
        assert float(dg.float().min()) == 3.0  # nothing was launched
        L.fln_set_static_scratch_limit(need)
        capi.layernorm_backward_static(x, x, st, st, None, x, dg, None)  # exactly at the limit: accepted
        torch.cuda.synchronize()
        assert float(dg.float().abs().max()) == 0.0
    finally:
        L.fln_set_static_scratch_limit(0)
