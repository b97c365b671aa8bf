"""GPU tests of the reference-facing Python surface (module, autograd Function, functional,
fused_layernorm_cuda.*), modelled on the reference's own tests/test_layernorm.py and its
script checks (tests/edge_cases.py, tests/prove_not_hardcoded.py, tests/break_kernel_test.py).
The oracle is the CPU checker on the same seeded inputs; torch.nn.LayerNorm on the GPU is
compared as well, at the reference's tolerances (1e-5 forward, 1e-4 gradients, fp16 1e-3)."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oracle import oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import fused_layernorm_cuda
    import gpu_util as U
    from fused_layernorm import (FusedLayerNorm, FusedLayerNormFunction, FusedRMSNorm, fused_add_layer_norm,
                                 fused_add_rms_norm, fused_add_rms_norm_fp8, fused_layer_norm, fused_rms_norm,
                                 replace_layernorm_modules)
    from fused_layernorm import _capi as capi
    from fused_layernorm.graphs import GraphedLayerNorm, GraphedLayerNormStep
    from fused_layernorm.hostio import HostLayerNormFwdBwd

F32, BF16, F16 = torch.float32, torch.bfloat16, torch.float16


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(42)


@pytest.mark.parametrize("batch,hidden,dtype", [(1, 768, F32), (8, 768, F32), (32, 1024, F32), (64, 2048, F32),
                                                (128, 4096, F32), (1, 768, F16), (32, 1024, F16), (64, 2048, F16),
                                                (32, 4096, BF16)])
def test_forward_correctness(batch, hidden, dtype):
    x = torch.randn(batch, hidden, device="cuda", dtype=dtype)
    ref = nn.LayerNorm(hidden, dtype=dtype).cuda()
    fused = FusedLayerNorm(hidden, dtype=dtype).cuda()
    with torch.no_grad():
        ref.weight.normal_(1, 0.1)
        ref.bias.normal_(0, 0.1)
        fused.load_state_dict(ref.state_dict())
    tol = 1e-5 if dtype == F32 else (1e-3 if dtype == F16 else 1.6e-2)
    got = fused(x)
    torch.testing.assert_close(got, ref(x), rtol=tol, atol=tol)
    want = O.norm_forward(x.cpu(), ref.weight.detach().cpu(), ref.bias.detach().cpu())["y"]
    U.assert_out_close(got.detach().cpu(), want, dtype)


@pytest.mark.parametrize("shape", [(2, 128, 768), (4, 256, 1024), (1, 1024, 4096), (2, 3, 5, 64)])
def test_nd_input(shape):
    x = torch.randn(*shape, device="cuda")
    ref = nn.LayerNorm(shape[-1]).cuda()
    fused = FusedLayerNorm(shape[-1]).cuda()
    out = fused(x)
    assert out.shape == x.shape
    torch.testing.assert_close(out, ref(x), rtol=1e-5, atol=1e-5)


def test_multi_dim_normalized_shape():
    x = torch.randn(6, 4, 32, device="cuda")
    ref = nn.LayerNorm((4, 32)).cuda()
    fused = FusedLayerNorm((4, 32)).cuda()
    with torch.no_grad():
        ref.weight.normal_()
        fused.load_state_dict(ref.state_dict())
    torch.testing.assert_close(fused(x), ref(x), rtol=1e-5, atol=1e-5)


def test_no_elementwise_affine():
    x = torch.randn(32, 1024, device="cuda")
    fused = FusedLayerNorm(1024, elementwise_affine=False).cuda()
    assert fused.weight is None and fused.bias is None
    torch.testing.assert_close(fused(x), F.layer_norm(x, (1024,)), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("batch,hidden", [(16, 768), (32, 1024), (64, 2048)])
def test_backward_correctness(batch, hidden):
    x = torch.randn(batch, hidden, device="cuda", requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    ref = nn.LayerNorm(hidden).cuda()
    fused = FusedLayerNorm(hidden).cuda()
    with torch.no_grad():
        ref.weight.normal_(1, 0.1)
        fused.load_state_dict(ref.state_dict())
    go = torch.randn(batch, hidden, device="cuda")
    ref(x).backward(go)
    fused(x2).backward(go)
    torch.testing.assert_close(x2.grad, x.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(fused.weight.grad, ref.weight.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(fused.bias.grad, ref.bias.grad, rtol=1e-4, atol=1e-4)


def test_gradient_accumulation():
    ref = nn.LayerNorm(1024).cuda()
    fused = FusedLayerNorm(1024).cuda()
    for _ in range(3):
        x = torch.randn(32, 1024, device="cuda")
        ref(x).sum().backward()
        fused(x).sum().backward()
    torch.testing.assert_close(fused.weight.grad, ref.weight.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(fused.bias.grad, ref.bias.grad, rtol=1e-4, atol=1e-4)


def test_needs_input_grad_masks():
    x = torch.randn(8, 256, device="cuda")  # no grad on input
    fused = FusedLayerNorm(256).cuda()
    fused.bias.requires_grad_(False)
    fused(x).sum().backward()
    assert fused.weight.grad is not None and fused.bias.grad is None


@pytest.mark.parametrize("eps", [1e-5, 1e-6, 1e-7, 1e-8])
def test_different_eps(eps):
    x = torch.randn(32, 1024, device="cuda")
    torch.testing.assert_close(FusedLayerNorm(1024, eps=eps).cuda()(x), nn.LayerNorm(1024, eps=eps).cuda()(x),
                               rtol=1e-5, atol=1e-5)


def test_determinism():
    fused = FusedLayerNorm(768).cuda()
    for seed in range(5):
        torch.manual_seed(seed)
        x = torch.randn(16, 768, device="cuda")
        outs = [fused(x) for _ in range(3)]
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("shape", [(1, 768), (32, 1), (2, 16384)])
def test_edge_shapes(shape):
    x = torch.randn(*shape, device="cuda")
    out = FusedLayerNorm(shape[-1]).cuda()(x)
    assert out.shape == x.shape
    torch.testing.assert_close(out, F.layer_norm(x, (shape[-1],)), rtol=1e-4, atol=1e-5)


def test_functional_interface():
    x = torch.randn(32, 1024, device="cuda")
    w, b = torch.randn(1024, device="cuda"), torch.randn(1024, device="cuda")
    torch.testing.assert_close(fused_layer_norm(x, (1024,), w, b, 1e-5), F.layer_norm(x, (1024,), w, b, 1e-5),
                               rtol=1e-5, atol=1e-5)
    x3 = torch.randn(4, 7, 1024, device="cuda")
    torch.testing.assert_close(fused_layer_norm(x3, 1024, w, b), F.layer_norm(x3, (1024,), w, b), rtol=1e-5, atol=1e-5)
    out = FusedLayerNormFunction.apply(x, (1024,), w, b, 1e-5)
    torch.testing.assert_close(out, F.layer_norm(x, (1024,), w, b), rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------- fused_layernorm_cuda.* (G2 + G1)
@pytest.mark.parametrize("shape", [(1, 1), (1, 17), (1000, 1), (1, 100000), (512, 512), (1, 32767), (1, 65536),
                                   (13, 13), (1, 4095), (1, 4097), (32, 4096)])
def test_g2_layernorm_positional_call(shape):
    x = torch.randn(*shape, device="cuda")
    ln = nn.LayerNorm(shape[1]).cuda()
    out = fused_layernorm_cuda.layernorm(x, ln.weight, ln.bias, 1e-5)
    assert torch.allclose(ln(x), out, rtol=1e-4, atol=1e-5)


def test_g2_keyword_forms_and_gelu():
    x = torch.randn(32, 4096, device="cuda")
    w, b = torch.randn(4096, device="cuda"), torch.randn(4096, device="cuda")
    base = fused_layernorm_cuda.layernorm(x, w, b, 1e-5)
    assert torch.equal(fused_layernorm_cuda.layernorm(x, w, b, eps=1e-5), base)          # README usage
    assert torch.equal(fused_layernorm_cuda.layernorm(input=x, gamma=w, beta=b, epsilon=1e-5), base)
    torch.testing.assert_close(fused_layernorm_cuda.layernorm(x, None, None, 1e-5), F.layer_norm(x, (4096,)),
                               rtol=1e-5, atol=1e-5)
    g_tanh = fused_layernorm_cuda.layernorm_gelu(x, w, b, 1e-5)                         # reference default: tanh form
    torch.testing.assert_close(g_tanh, F.gelu(F.layer_norm(x, (4096,), w, b), approximate="tanh"), rtol=1e-5, atol=1e-5)
    g_erf = fused_layernorm_cuda.layernorm_gelu(x, w, b, 1e-5, approximate="none")
    torch.testing.assert_close(g_erf, F.gelu(F.layer_norm(x, (4096,), w, b)), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(torch.ops.fused_layernorm.layernorm_gelu(x, w, b, 1e-5, "tanh"), g_tanh)


def test_g2_rejects_what_the_reference_silently_misreads():
    x = torch.randn(32, 4096, device="cuda")
    with pytest.raises(RuntimeError, match="size must match hidden dimension"):       # tests/prove_not_hardcoded.py:63-78
        fused_layernorm_cuda.layernorm(x, torch.ones(4095, device="cuda"), torch.zeros(4095, device="cuda"), 1e-5)
    with pytest.raises(NotImplementedError, match="not implemented for 'Double'"):      # tests/break_kernel_test.py:44-51
        fused_layernorm_cuda.layernorm(x.double(), None, None, 1e-5)
    with pytest.raises(RuntimeError, match="2D"):
        fused_layernorm_cuda.layernorm(x.view(2, 16, 4096), None, None, 1e-5)
    with pytest.raises(RuntimeError, match="same dtype"):
        fused_layernorm_cuda.layernorm(x, torch.ones(4096, device="cuda", dtype=F16), None, 1e-5)
    xt = torch.randn(4096, 32, device="cuda").t()                                       # non-contiguous: copied, not misread
    torch.testing.assert_close(fused_layernorm_cuda.layernorm(xt, None, None, 1e-5), F.layer_norm(xt, (4096,)),
                               rtol=1e-5, atol=1e-5)
    out = fused_layernorm_cuda.layernorm(x, None, None, 1e-12)                          # tests/break_kernel_test.py:39-41
    assert torch.allclose(out, F.layer_norm(x, (4096,), eps=1e-12), rtol=1e-4, atol=1e-5)


def test_g1_forward_backward_signatures():
    x = torch.randn(48, 1024, device="cuda")
    w, b = torch.randn(1024, device="cuda"), torch.randn(1024, device="cuda")
    dy = torch.randn_like(x)
    out, mean, rstd = fused_layernorm_cuda.forward(x, w, b, 1e-5)
    o2, m2, r2 = fused_layernorm_cuda.forward(input=x, gamma=w, beta=b)
    assert torch.equal(out, o2) and mean.dtype == torch.float32 and mean.shape == (48,)
    t_out, t_mean, t_rstd = torch.native_layer_norm(x, (1024,), w, b, 1e-5)
    torch.testing.assert_close(mean, t_mean.reshape(-1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rstd, t_rstd.reshape(-1), rtol=1e-5, atol=1e-5)
    dx, dg, db = fused_layernorm_cuda.backward(dy, x, mean, rstd, w, b, [True, True, True])
    tdx, tdg, tdb = torch.ops.aten.native_layer_norm_backward(dy, x, [1024], t_mean, t_rstd, w, b, [True, True, True])
    torch.testing.assert_close(dx, tdx, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(dg, tdg, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(db, tdb, rtol=1e-4, atol=1e-4)
    dx2, dg2, db2 = fused_layernorm_cuda.backward(dy, x, mean, rstd, w, b, output_mask=[True, False, False])
    assert dg2 is None and db2 is None and torch.equal(dx2, dx)
    dx3, dg3, db3 = fused_layernorm_cuda.backward(dy, x, mean, rstd)                    # no gamma/beta: no param grads
    assert dg3 is None and db3 is None


# ------------------------------------------------------------------------- additions
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_rmsnorm_module_and_grads(dtype):
    x = torch.randn(4, 33, 512, device="cuda", dtype=dtype, requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    ref = nn.RMSNorm(512, eps=1e-6, dtype=dtype).cuda()
    fused = FusedRMSNorm(512, eps=1e-6, dtype=dtype).cuda()
    with torch.no_grad():
        ref.weight.normal_(1, 0.1)
        fused.load_state_dict(ref.state_dict())
    go = torch.randn_like(x)
    ref(x).backward(go)
    fused(x2).backward(go)
    tol = 1e-4 if dtype == F32 else 3e-2
    torch.testing.assert_close(fused(x2), ref(x), rtol=tol, atol=tol)
    torch.testing.assert_close(x2.grad, x.grad, rtol=tol, atol=tol)
    torch.testing.assert_close(fused.weight.grad.float(), ref.weight.grad.float(), rtol=3e-2, atol=3e-2 * (33 * 4) ** 0.5)
    want = O.norm_forward(x.detach().cpu().reshape(-1, 512), ref.weight.detach().cpu(), None, None, "rmsnorm", 1e-6)["y"]
    U.assert_out_close(fused(x2).detach().cpu().reshape(-1, 512), want, dtype)


def test_fused_add_norm_autograd_includes_residual_stream_gradient():
    x = torch.randn(64, 1024, device="cuda", requires_grad=True)
    r = torch.randn(64, 1024, device="cuda", requires_grad=True)
    w = torch.randn(1024, device="cuda", requires_grad=True)
    b = torch.randn(1024, device="cuda", requires_grad=True)
    x2, r2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, r, w, b))
    gy, gs = torch.randn(64, 1024, device="cuda"), torch.randn(64, 1024, device="cuda")
    y, s = fused_add_layer_norm(x, r, w, b, 1e-5)
    (y * gy + s * gs).sum().backward()
    s_ref = x2 + r2
    y_ref = F.layer_norm(s_ref, (1024,), w2, b2, 1e-5)
    (y_ref * gy + s_ref * gs).sum().backward()
    torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-5)
    assert torch.equal(s, s_ref)
    for a, c in ((x.grad, x2.grad), (r.grad, r2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-4)
    # only the sum is used downstream
    x3 = x.detach().clone().requires_grad_(True)
    _, s3 = fused_add_rms_norm(x3, r.detach(), w.detach())
    s3.sum().backward()
    assert torch.equal(x3.grad, torch.ones_like(x3))


def test_fp8_function():
    x = torch.randn(256, 2048, device="cuda", dtype=BF16)
    r = (0.5 * torch.randn(256, 2048, device="cuda")).to(BF16)
    w = (1 + 0.1 * torch.randn(2048, device="cuda")).to(BF16)
    q, s, scale = fused_add_rms_norm_fp8(x, r, w, 1e-6)
    assert q.dtype == torch.float8_e4m3fn and scale.shape == (1,) and torch.equal(s, x + r)
    want = O.norm_forward(x.cpu(), w.cpu(), None, r.cpu(), "rmsnorm", 1e-6)
    wq, wamax, wscale = O.quant_fp8(want["y32"])
    torch.testing.assert_close(scale.cpu(), wscale, rtol=1e-5, atol=0)
    d = O.fp8_code_distance(q.view(torch.uint8).cpu(), wq)
    assert int(d.max()) <= 1 and int((d > 0).sum()) <= max(1, int(1e-4 * d.numel()))
    q2, s2, _ = fused_layernorm_cuda.add_rmsnorm_fp8(x, None, w, 1e-6)
    assert q2.shape == x.shape and s2.numel() == 0


def test_fp8_one_pass_functions():
    from fused_layernorm import fused_add_norm_fp8_delayed, fused_add_norm_fp8_rowwise
    x = torch.randn(4, 64, 2048, device="cuda", dtype=BF16)
    r = (0.5 * torch.randn(4, 64, 2048, device="cuda")).to(BF16)
    w = (1 + 0.1 * torch.randn(2048, device="cuda")).to(BF16)
    want = O.norm_forward(x.cpu().reshape(-1, 2048), w.cpu(), None, r.cpu().reshape(-1, 2048), "rmsnorm", 1e-6)
    # step 0 measures amax with a neutral scale, step 1 quantizes with 448 / that amax
    _, _, amax = fused_add_norm_fp8_delayed(x, torch.ones(1, device="cuda"), r, w)
    torch.testing.assert_close(amax.cpu(), want["y32"].abs().max().reshape(1), rtol=1e-5, atol=0)
    scale = 448.0 / amax
    q, s, amax2 = fused_add_norm_fp8_delayed(x, scale, r, w)
    assert q.shape == x.shape and q.dtype == torch.float8_e4m3fn and torch.equal(s, x + r) and torch.equal(amax, amax2)
    wq, _ = O.quant_fp8_delayed(want["y32"], scale.cpu())
    d = O.fp8_code_distance(q.view(torch.uint8).cpu().reshape(-1, 2048), wq)
    assert int(d.max()) <= 1 and int((d > 0).sum()) <= max(1, int(1e-4 * d.numel()))
    q, s, rs = fused_add_norm_fp8_rowwise(x, r, w)
    assert rs.shape == (256,) and torch.equal(s, x + r)
    deq = q.float().reshape(-1, 2048).cpu() / rs.cpu()[:, None]
    assert bool(((deq - want["y32"]).abs() <= want["y32"].abs() * 0.0625 + (2.0 ** -9 / rs.cpu())[:, None]).all())
    q3, s3, rs3 = fused_add_norm_fp8_rowwise(x, None, w, None, 1e-5, "layernorm")
    assert s3 is None and rs3.shape == (256,)


def test_mxfp8_function_dequantizes_to_the_normalized_values():
    from fused_layernorm import fused_add_norm_mxfp8
    x = torch.randn(4, 64, 2048, device="cuda", dtype=BF16) * 3
    r = (0.5 * torch.randn(4, 64, 2048, device="cuda")).to(BF16)
    w = (1 + 0.1 * torch.randn(2048, device="cuda")).to(BF16)
    q, s, scales = fused_add_norm_mxfp8(x, r, w)
    assert q.shape == x.shape and q.dtype == torch.float8_e4m3fn and scales.shape == (4, 64, 64)
    assert torch.equal(s, x + r)
    want = O.norm_forward(x.cpu().reshape(-1, 2048), w.cpu(), None, r.cpu().reshape(-1, 2048), "rmsnorm", 1e-6)["y32"]
    e = scales.view(torch.uint8).cpu().reshape(-1, 64).to(torch.float64)
    deq = (q.float().cpu().reshape(-1, 64, 32).double() * torch.pow(2.0, e - 127)[..., None]).reshape(-1, 2048)
    # e4m3 keeps 3 mantissa bits and the block maximum is scaled into [256, 512): the error is at
    # most half a step of the element's binade, and one step (32 * scale) where it saturates
    step = torch.pow(2.0, e - 127)[..., None].expand(-1, -1, 32).reshape(-1, 2048)
    err = (deq - want.double()).abs()
    assert bool((err <= want.abs().double() * 0.0625 + 64 * step).all())
    assert float((err / (want.abs().double() + 1e-3)).median()) < 0.04


def test_replace_layernorm_modules_on_device():
    model = nn.Sequential(nn.Linear(256, 256), nn.LayerNorm(256), nn.GELU(), nn.LayerNorm(256)).cuda()
    x = torch.randn(16, 256, device="cuda")
    want = model(x)
    assert replace_layernorm_modules(model) == 2
    torch.testing.assert_close(model(x), want, rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------ tracing / graphs / host path
def test_torch_compile_traces_the_module_without_graph_breaks():
    fused = FusedLayerNorm(1024).cuda()
    x = torch.randn(32, 1024, device="cuda", requires_grad=True)
    compiled = torch.compile(fused, backend="aot_eager", fullgraph=True)
    out = compiled(x)
    torch.testing.assert_close(out, fused(x), rtol=0, atol=0)
    out.sum().backward()
    assert x.grad is not None and fused.weight.grad is not None

    def block(a, res, w):
        y, s = fused_add_rms_norm(a, res, w)
        return fused_rms_norm(y, w) + s

    a, res, w = torch.randn(8, 512, device="cuda"), torch.randn(8, 512, device="cuda"), torch.randn(512, device="cuda")
    torch.testing.assert_close(torch.compile(block, backend="aot_eager", fullgraph=True)(a, res, w), block(a, res, w))


def test_opcheck_layernorm_fwd():
    x = torch.randn(8, 256, device="cuda", requires_grad=True)
    w = torch.randn(256, device="cuda", requires_grad=True)
    b = torch.randn(256, device="cuda", requires_grad=True)
    torch.library.opcheck(torch.ops.fused_layernorm.layernorm_fwd.default, (x, w, b, 1e-5),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_composes_with_torch_cuda_graph_capture():
    fused = FusedLayerNorm(4096).cuda()
    x = torch.randn(32, 4096, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s), torch.no_grad():
        for _ in range(3):
            fused(x)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(g):
        y = fused(x)
    x.copy_(torch.randn(32, 4096, device="cuda"))
    g.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(y, F.layer_norm(x, (4096,), fused.weight, fused.bias), rtol=1e-5, atol=1e-5)


def test_own_graph_path():
    x = torch.randn(32, 4096, device="cuda")
    w, b = torch.randn(4096, device="cuda"), torch.randn(4096, device="cuda")
    g = GraphedLayerNorm(x, w, b, 1e-5, repeat=4)
    x.copy_(torch.randn_like(x))
    y = g()
    torch.cuda.synchronize()
    torch.testing.assert_close(y, F.layer_norm(x, (4096,), w, b), rtol=1e-5, atol=1e-5)
    g.close()
    dy = torch.randn_like(x)
    st = GraphedLayerNormStep(x, dy, w, b)
    y, dx, dw, db = st()
    torch.cuda.synchronize()
    xr = x.clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    F.layer_norm(xr, (4096,), wr, br).backward(dy)
    torch.testing.assert_close(dx, xr.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(dw, wr.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(db, br.grad, rtol=1e-4, atol=1e-4)
    st.close()


def test_graph_replay_of_the_pipelined_step_with_fused_column_reduce():
    """A shape served by the persistent pipeline: the backward is a cooperative launch whose
    tail synchronises the grid on a workspace word tagged with a launch token.  A captured graph
    replays the same token, so the word has to come back clean after every replay; three
    replays with fresh inputs, in the library's own graph and in torch's, against eager calls."""
    rows, cols = 8192, 4096
    x = torch.randn(rows, cols, device="cuda", dtype=BF16)
    dy = torch.randn_like(x)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(BF16)
    b = (0.1 * torch.randn(cols, device="cuda")).to(BF16)
    assert capi.describe_launch(True, rows, cols, BF16)["pipelined"] == 1

    def eager():
        y, mean, rstd = torch.empty_like(x), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
        dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)
        ws = torch.empty(capi.backward_workspace_bytes(rows, cols, BF16) // 4, device="cuda")
        capi.layernorm_forward(x, w, b, y, mean, rstd, 1e-5)
        capi.layernorm_backward(dy, x, mean, rstd, w, dx, dw, db, ws)
        return y, dx, dw, db

    st = GraphedLayerNormStep(x, dy, w, b)
    for _ in range(3):
        x.copy_(torch.randn_like(x))
        dy.copy_(torch.randn_like(dy))
        got = [t.clone() for t in st()]
        want = eager()
        torch.cuda.synchronize()
        for g_, w_ in zip(got, want):
            assert torch.equal(g_, w_)
    st.close()

    y, mean, rstd = torch.empty_like(x), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)
    ws = torch.empty(capi.backward_workspace_bytes(rows, cols, BF16) // 4, device="cuda")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        capi.layernorm_forward(x, w, b, y, mean, rstd, 1e-5)
        capi.layernorm_backward(dy, x, mean, rstd, w, dx, dw, db, ws)
    for _ in range(3):
        x.copy_(torch.randn_like(x))
        g.replay()
        want = eager()
        torch.cuda.synchronize()
        assert torch.equal(dx, want[1]) and torch.equal(dw, want[2]) and torch.equal(db, want[3])
    assert capi.lib().fln_device_status() == 0


def test_host_pipelined_path_matches_device_path():
    rows, cols = 4096 + 100, 1024
    x, gamma, beta, dy, _ = U.make_inputs(5, rows, cols, BF16)
    pipe = HostLayerNormFwdBwd(rows, cols, BF16, chunk_rows=1024)
    xh, dyh = x.pin_memory(), dy.pin_memory()
    yh, dxh = torch.empty_like(x).pin_memory(), torch.empty_like(x).pin_memory()
    dph = torch.empty(2 * cols, dtype=BF16).pin_memory()
    pipe(xh, dyh, gamma.cuda(), beta.cuda(), yh, dxh, dph)
    torch.cuda.synchronize()
    f = O.norm_forward(x, gamma, beta)
    b = O.norm_backward(dy, x, f["mean"], f["rstd"], gamma)
    U.assert_out_close(yh, f["y"], BF16)
    U.assert_out_close(dxh, b["dx"], BF16)
    assert int(O.mismatch_16(dph[:cols], b["dgamma"], abs_floor=2e-2).sum()) == 0
    assert int(O.mismatch_16(dph[cols:], b["dbeta"], abs_floor=2e-2).sum()) == 0
