"""NVFP4-style block-scaled 4-bit output (e2m1 elements, e4m3 scale per 16 elements, fp32 tensor
scale) of the fused residual-add + norm forward, through the C ABI, against the CPU checker."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as U
    from fused_layernorm import _capi as capi
    from oracle import oracle as O

BF16, F32 = torch.bfloat16, torch.float32


def _nibbles(q):
    return torch.stack([q & 15, q >> 4], dim=-1).reshape(q.shape[0], -1).to(torch.int32)


def _e2m1_distance(a, b):
    """distance in code steps between e2m1 codes (sign-magnitude order; +0 and -0 coincide)"""
    key = lambda c: torch.where(c >= 8, -(c - 8), c)
    return (key(_nibbles(a)) - key(_nibbles(b))).abs()


@pytest.mark.parametrize("shape", [(64, 1024), (33, 4096), (48, 8192), (5, 16), (40, 1600)])
@pytest.mark.parametrize("dtype", [BF16, F32])
@pytest.mark.parametrize("kind,residual", [("rmsnorm", True), ("layernorm", False)])
def test_nvfp4_block_scaled_output(shape, dtype, kind, residual):
    rows, cols = shape
    x, gamma, beta, _, res = U.make_inputs(20248, rows, cols, dtype, residual=residual, outliers=True)
    if kind == "rmsnorm":
        beta = None
    want = O.norm_forward(x, gamma, beta, res, kind, 1e-6)
    y32 = want["y32"]
    S = 448.0 * 6.0 / float(y32.abs().max()) * 0.9  # a scale from "the previous step": close, not exact
    q = U.Guarded((rows, cols // 2), torch.uint8)
    bs = U.Guarded((rows, cols // 16), torch.uint8)
    s = U.Guarded((rows, cols), dtype) if residual else None
    amax = torch.full((1,), -1.0, device="cuda")
    capi.norm_forward_nvfp4(U.KINDS[kind], U.dev(x), U.dev(res), U.dev(gamma), U.dev(beta), q.t, bs.t,
                            s.t if s else None, None, None, torch.tensor([S], device="cuda"), amax, 1e-6)
    torch.cuda.synchronize()
    got_q, got_bs = q.check().cpu(), bs.check().cpu()
    _, want_bs = O.quant_nvfp4(y32, S)
    # block scales: e4m3 codes, at most one code step apart, and only on a few blocks (where the
    # block maximum times S / 6 sits within rounding of a tie)
    dbs = O.fp8_code_distance(got_bs, want_bs)
    assert int(dbs.max()) <= 1 and int((dbs > 0).sum()) <= max(1, int(2e-3 * dbs.numel()))
    # elements against the quantizer run with the device's own block scales
    wq, _ = O.quant_nvfp4(y32, S, got_bs)
    d = _e2m1_distance(got_q, wq)
    assert int(d.max()) <= 1 and int((d > 0).sum()) <= max(1, int(2e-4 * d.numel()))
    # and the round trip reproduces y within half a step of the block's grid
    deq = O.dequant_nvfp4(got_q, got_bs, S)
    e4 = torch.tensor([O.lib().oracle_e4m3_decode(c) for c in range(256)])
    step = (e4[got_bs.long()] / S).repeat_interleave(16, dim=1)  # value of one e2m1 unit in this block
    assert bool(((deq - y32).abs() <= 1.0 * step + 1e-6).all())
    torch.testing.assert_close(amax.cpu(), y32.abs().max().reshape(1), rtol=1e-5, atol=0)
    if residual:
        assert torch.equal(s.check().cpu().view(torch.uint8), want["sum"].view(torch.uint8))


@pytest.mark.parametrize("shape", [(1024, 8192), (768, 3072), (2048, 1024), (2051, 1024), (1031, 4096)])
@pytest.mark.parametrize("dtype", [BF16, torch.float16])
@pytest.mark.parametrize("kind,residual", [("rmsnorm", True), ("layernorm", False)])
def test_nvfp4_through_the_pipelined_forward(shape, dtype, kind, residual):
    """The same checks with the persistent pipelined forward doing the work (forced for these
    medium sizes; large 16-bit problems take it by themselves)."""
    capi.lib().fln_set_path_override(2)
    try:
        test_nvfp4_block_scaled_output(shape, dtype, kind, residual)
        assert capi.lib().fln_device_status() == 0
    finally:
        capi.lib().fln_set_path_override(0)


def test_nvfp4_python_api_and_errors():
    import fused_layernorm as fl
    x = torch.randn(2, 8, 256, device="cuda", dtype=BF16)
    w = torch.ones(256, device="cuda", dtype=BF16)
    S = torch.tensor([448.0 * 6.0 / 4.0], device="cuda")
    q, bs, amax, s = fl.fused_add_norm_nvfp4(x, S, residual=x, weight=w)
    assert q.shape == (2, 8, 128) and bs.shape == (2, 8, 16) and s.shape == x.shape and amax.shape == (1,)
    with pytest.raises(RuntimeError):
        capi.norm_forward_nvfp4(capi.RMSNORM, x.reshape(16, 256)[:, :24].contiguous(), None, None, None,
                                torch.empty(16, 12, dtype=torch.uint8, device="cuda"),
                                torch.empty(16, 2, dtype=torch.uint8, device="cuda"), None, None, None, S, None, 1e-6)
