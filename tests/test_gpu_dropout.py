"""Fused dropout -> residual add -> norm forward and the dropout backward, through the C ABI,
against the CPU checker: the mask must be bit for bit the Philox mask of (seed, offset), the
outputs those of the unfused composition on that mask (dropout rounded to the I/O type, sum
rounded to the I/O type, norm), and the gradient of x the masked, scaled gradient of the sum."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as U
    from fused_layernorm import _capi as capi
    from oracle import oracle as O

BF16, F16, F32 = torch.bfloat16, torch.float16, torch.float32


@pytest.mark.parametrize("rows,cols,dtype", [(64, 1024, BF16), (33, 1000, BF16), (256, 8192, BF16), (48, 4096, F32),
                                             (17, 16384, F16), (5, 8, F32), (40, 1600, BF16)])
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
@pytest.mark.parametrize("p", [0.1, 0.0])
def test_dropout_add_norm_forward(rows, cols, dtype, kind, p):
    x, gamma, beta, dy, res = U.make_inputs(41, rows, cols, dtype, residual=True)
    if kind == "rmsnorm":
        beta = None
    seed, offset = 0x1234567890abcdef, 3
    d = lambda t: None if t is None else t.cuda()
    y, s = U.Guarded((rows, cols), dtype), U.Guarded((rows, cols), dtype)
    mean = U.Guarded((rows,), F32) if kind == "layernorm" else None
    rstd = U.Guarded((rows,), F32)
    bits = U.Guarded((rows * cols // 8,), torch.uint8)
    capi.dropout_add_norm_forward(U.KINDS[kind], d(x), d(res), d(gamma), d(beta), y.t, s.t, mean.t if mean else None,
                                  rstd.t, bits.t, 1e-5, p, seed, offset)
    torch.cuda.synchronize()
    want_bits = O.dropout_keep_bits(seed, offset, p, rows * cols)
    assert torch.equal(bits.check().cpu(), want_bits)
    dropped = O.dropout_apply(x, want_bits, p)
    if p == 0.0:
        assert torch.equal(dropped, x)
    w = O.norm_forward(dropped, gamma, beta, residual=res, kind=kind)
    assert torch.equal(s.check().cpu(), w["sum"])  # the residual stream is exact
    U.assert_out_close(y.check().cpu(), w["y"], dtype)
    torch.testing.assert_close(rstd.check().cpu(), w["rstd"], rtol=1e-5, atol=1e-5)
    if mean:
        torch.testing.assert_close(mean.check().cpu(), w["mean"], rtol=1e-5, atol=1e-5)


def test_dropout_without_residual_and_without_stored_mask():
    rows, cols = 128, 2048
    x, gamma, beta, dy, _ = U.make_inputs(42, rows, cols, BF16)
    y = torch.empty(rows, cols, dtype=BF16, device="cuda")
    capi.dropout_add_norm_forward(capi.LAYERNORM, x.cuda(), None, gamma.cuda(), beta.cuda(), y, None, None, None, None,
                                  1e-5, 0.25, 5, 0)
    torch.cuda.synchronize()
    bits = O.dropout_keep_bits(5, 0, 0.25, rows * cols)
    w = O.norm_forward(O.dropout_apply(x, bits, 0.25), gamma, beta)
    U.assert_out_close(y.cpu(), w["y"], BF16)


@pytest.mark.parametrize("rows,cols,dtype", [(1024, 8192, BF16), (2048, 1024, F16), (768, 3072, BF16), (512, 16384, BF16),
                                             (1200, 768, F16), (2051, 1024, BF16), (1031, 4096, F16), (1203, 768, BF16)])
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
@pytest.mark.parametrize("p", [0.1, 0.0])
def test_dropout_through_the_pipelined_forward(rows, cols, dtype, kind, p):
    """Large 16-bit problems run with the dropout folded into the persistent pipelined forward
    (forced here for medium sizes): same mask bits, same residual stream, same checks; also
    without a residual, with and without the dropped x written out.  Row counts that do not fill
    the plan's row slots (2051, 1031, 1203) leave their last rows to the one-row-per-CTA kernel,
    which draws the mask bits of the rows' place in the whole tensor."""
    capi.lib().fln_set_path_override(2)
    try:
        test_dropout_add_norm_forward(rows, cols, dtype, kind, p)
        x, gamma, beta, dy, _ = U.make_inputs(43, rows, cols, dtype)
        if kind == "rmsnorm":
            beta = None
        d = lambda t: None if t is None else t.cuda()
        bits = O.dropout_keep_bits(7, 11, p, rows * cols)
        dropped = O.dropout_apply(x, bits, p)
        w = O.norm_forward(dropped, gamma, beta, kind=kind)
        for with_sum in (True, False):
            y = U.Guarded((rows, cols), dtype)
            s = U.Guarded((rows, cols), dtype) if with_sum else None
            capi.dropout_add_norm_forward(U.KINDS[kind], d(x), None, d(gamma), d(beta), y.t, s.t if s else None, None,
                                          None, None, 1e-5, p, 7, 11)
            torch.cuda.synchronize()
            U.assert_out_close(y.check().cpu(), w["y"], dtype)
            if with_sum:
                assert torch.equal(s.check().cpu(), dropped)
        assert capi.lib().fln_device_status() == 0
    finally:
        capi.lib().fln_set_path_override(0)


@pytest.mark.parametrize("dtype", [BF16, F32])
@pytest.mark.parametrize("stored", [True, False])
def test_dropout_backward_from_stored_or_regenerated_mask(dtype, stored):
    rows, cols, p, seed, offset = 96, 4096, 0.3, 77, 11
    g = torch.Generator().manual_seed(43)
    ds = torch.randn(rows, cols, generator=g).to(dtype)
    bits = O.dropout_keep_bits(seed, offset, p, rows * cols)
    dx = U.Guarded((rows, cols), dtype)
    capi.dropout_backward(ds.cuda(), bits.cuda() if stored else None, dx.t, p, seed, offset)
    torch.cuda.synchronize()
    assert torch.equal(dx.check().cpu(), O.dropout_apply(ds, bits, p))


def test_whole_block_gradients_match_autograd_on_the_unfused_composition():
    """d(dropout -> add -> layernorm) / d(x, residual, gamma, beta) from the library's pieces
    (norm backward on (dy, s), dropout backward) against torch autograd on the same mask."""
    rows, cols, p, seed, offset = 64, 1024, 0.2, 9, 1
    x, gamma, beta, dy, res = U.make_inputs(44, rows, cols, F32, residual=True)
    d = lambda t: t.cuda()
    y, s = torch.empty(rows, cols, device="cuda"), torch.empty(rows, cols, device="cuda")
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    bits = torch.empty(rows * cols // 8, dtype=torch.uint8, device="cuda")
    capi.dropout_add_norm_forward(capi.LAYERNORM, d(x), d(res), d(gamma), d(beta), y, s, mean, rstd, bits, 1e-5, p, seed, offset)
    ds = torch.empty(rows, cols, device="cuda")
    dgb = torch.empty(2 * cols, device="cuda")
    ws = torch.empty(max(capi.backward_workspace_bytes(rows, cols, F32) // 4, 1), device="cuda")
    capi.norm_backward(capi.LAYERNORM, d(dy), s, mean, rstd, d(gamma), None, ds, None, None, dgb, ws)
    dxx = torch.empty(rows, cols, device="cuda")
    capi.dropout_backward(ds, bits, dxx, p, seed, offset)
    torch.cuda.synchronize()
    # autograd reference in float64 with the kernel's own mask
    keep = torch.tensor(__import__("numpy").unpackbits(bits.cpu().numpy(), bitorder="little")).reshape(rows, cols).double()
    _, scale = O.dropout_threshold(p)
    xr, rr = x.double().requires_grad_(True), res.double().requires_grad_(True)
    gr, br = gamma.double().requires_grad_(True), beta.double().requires_grad_(True)
    out = torch.nn.functional.layer_norm(xr * keep * scale + rr, (cols,), gr, br, 1e-5)
    out.backward(dy.double())
    torch.testing.assert_close(y.cpu().double(), out.detach(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ds.cpu().double(), rr.grad, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(dxx.cpu().double(), xr.grad, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(dgb.cpu().double(), torch.cat([gr.grad, br.grad]), rtol=1e-4, atol=1e-4)


def test_dropout_argument_errors():
    x = torch.zeros(4, 16, dtype=BF16, device="cuda")
    with pytest.raises(RuntimeError):
        capi.dropout_add_norm_forward(capi.LAYERNORM, x, None, None, None, x, None, None, None, None, 1e-5, 1.0, 1, 0)  # p = 1
    with pytest.raises(RuntimeError):
        capi.dropout_add_norm_forward(capi.LAYERNORM, x[:, :12].contiguous(), None, None, None, x, None, None, None, None,
                                      1e-5, 0.1, 1, 0)  # cols % 8


def test_python_api_is_differentiable_and_reproducible():
    import fused_layernorm as fl
    torch.manual_seed(123)
    rows, cols = 32, 512
    x = torch.randn(2, rows // 2, cols, device="cuda", requires_grad=True)
    res = torch.randn(2, rows // 2, cols, device="cuda", requires_grad=True)
    w = torch.randn(cols, device="cuda", requires_grad=True)
    b = torch.randn(cols, device="cuda", requires_grad=True)
    y, s = fl.fused_dropout_add_layer_norm(x, res, w, b, p=0.25, seed=11, offset=4)
    y2, s2 = fl.fused_dropout_add_layer_norm(x, res, w, b, p=0.25, seed=11, offset=4)
    assert torch.equal(y, y2) and torch.equal(s, s2)
    y3, _ = fl.fused_dropout_add_layer_norm(x, res, w, b, p=0.25, seed=11, offset=5)
    assert not torch.equal(y, y3)
    (y.sum() + 0.5 * s.sum()).backward()
    # reference: autograd through the unfused composition with the same mask
    bits = O.dropout_keep_bits(11, 4, 0.25, rows * cols)
    keep = torch.tensor(__import__("numpy").unpackbits(bits.numpy(), bitorder="little")).reshape(x.shape).double().cuda()
    _, scale = O.dropout_threshold(0.25)
    xr, rr, wr, br = (t.detach().double().requires_grad_(True) for t in (x, res, w, b))
    sr = xr * keep * scale + rr
    yr = torch.nn.functional.layer_norm(sr, (cols,), wr, br, 1e-5)
    (yr.sum() + 0.5 * sr.sum()).backward()
    torch.testing.assert_close(y.double(), yr.detach(), rtol=1e-5, atol=2e-5)
    for got, want in ((x.grad, xr.grad), (res.grad, rr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-4)
    # evaluation mode drops nothing
    ye, se = fl.fused_dropout_add_layer_norm(x, res, w, b, p=0.25, training=False)
    torch.testing.assert_close(se, x + res)
