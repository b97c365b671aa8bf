"""Pins the CPU oracle (oracle/fln_oracle.c) against the frozen torch-CPU fixtures.

Tolerances: fp32 results 1e-5 abs/rel (the bar the reference's tests use,
tests/test_layernorm.py:32-33 of the reference; observed differences are ~1e-6); bf16 / fp16
results at most 1 unit in the last place (or 1e-5 absolute where the value is a
near-zero difference, see oracle.mismatch_16); fp8 codes at most one code step on at most 0.01 % of
the elements; element conversions bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O

CASES = ["c1_ln_f32_32x768", "c2_ln_f32_5x1023", "c2_ln_bf16_5x1023", "c2_ln_bf16_2x4096",
         "ln_f16_8x256", "c3_addln_bf16_8x512", "c4_addrms_fp8_bf16_8x1024", "rms_f32_8x384",
         "ln_f32_noaffine_5x13"]


def close32(a, b, tol=1e-5):
    torch.testing.assert_close(a.float(), b.float(), rtol=tol, atol=tol)


def close_out(a, b, dtype):
    if dtype == torch.float32:
        close32(a, b)
    else:
        assert int(O.mismatch_16(a, b).sum()) == 0


def test_golden_has_all_cases(golden):
    assert set(CASES) <= set(golden.names)


@pytest.mark.parametrize("name", CASES)
def test_forward_matches_torch_cpu(golden, name):
    c = golden.case(name)
    r = O.norm_forward(c["x"], c["gamma"], c["beta"], c["res"], c["kind"], c["eps"])
    close_out(r["y"], c["y"], c["dtype"])
    close32(r["rstd"], c["rstd"], 2e-6)
    if c["kind"] == "layernorm":
        close32(r["mean"], c["mean"], 2e-6)
    if c["res"] is not None:
        assert torch.equal(r["sum"].view(torch.int16), c["sum"].view(torch.int16))
    for act in ("gelu_tanh", "gelu_erf"):
        if "y_" + act in c:
            ra = O.norm_forward(c["x"], c["gamma"], c["beta"], None, c["kind"], c["eps"], act)
            close_out(ra["y"], c["y_" + act], c["dtype"])


@pytest.mark.parametrize("name", CASES)
def test_backward_matches_torch_autograd(golden, name):
    c = golden.case(name)
    f = O.norm_forward(c["x"], c["gamma"], c["beta"], c["res"], c["kind"], c["eps"])
    s = f["sum"] if c["res"] is not None else c["x"]
    b = O.norm_backward(c["dy"], s, f["mean"], f["rstd"], c["gamma"], None, c["kind"])
    # the fixture's dx is float64 autograd rounded to fp32; the oracle uses fp32 saved stats
    torch.testing.assert_close(b["dx32"], c["dx"], rtol=2e-5, atol=2e-5)
    if c["dgamma"] is not None:
        torch.testing.assert_close(b["dgamma64"].float(), c["dgamma"], rtol=1e-5, atol=1e-5)
    if c["dbeta"] is not None:
        torch.testing.assert_close(b["dbeta64"].float(), c["dbeta"], rtol=1e-5, atol=1e-5)


def test_fp8_quantization_matches_torch_cast(golden):
    c = golden.case("c4_addrms_fp8_bf16_8x1024")
    f = O.norm_forward(c["x"], c["gamma"], None, c["res"], "rmsnorm", c["eps"])
    q, amax, scale = O.quant_fp8(f["y32"])
    torch.testing.assert_close(amax, c["amax"], rtol=1e-6, atol=0)
    torch.testing.assert_close(scale, c["scale"], rtol=1e-6, atol=0)
    d = O.fp8_code_distance(q, c["q"])
    assert int(d.max()) <= 1
    assert float((d > 0).float().mean()) <= 1e-4
    # on identical fp32 inputs the encoder itself is bit-exact
    q2, _, _ = O.quant_fp8(c["y32"])
    assert torch.equal(q2, c["q"])


def test_conversions_bit_exact(golden):
    src = torch.from_numpy(golden.raw("convert/src").copy())
    bf = O.convert_from_f32(src, torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bf, golden.raw("convert/bf16"))
    f16 = O.convert_from_f32(src, torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(f16, golden.raw("convert/f16"))
    e = O.e4m3_encode(torch.from_numpy(golden.raw("convert/e4m3_src").copy())).numpy()
    assert np.array_equal(e, golden.raw("convert/e4m3"))


def test_stability_rows(golden):
    """Constant 1e-8 / 1e8 rows and randn*1e-4 / 1e4 rows (reference tests/test_layernorm.py:238-270)."""
    x = torch.from_numpy(golden.raw("stability/x").copy())
    y = O.norm_forward(x, None, None, None, "layernorm", 1e-5)["y"]
    assert torch.isfinite(y).all()
    torch.testing.assert_close(y, torch.from_numpy(golden.raw("stability/y").copy()), rtol=1e-3, atol=1e-3)


def test_literal_g2_restatement_agrees_with_truth(golden):
    """The order-faithful fp32 restatement and the double-accumulator oracle agree to 1e-5."""
    c = golden.case("c1_ln_f32_32x768")
    y = O.ref_g2_layernorm(c["x"], c["gamma"], c["beta"], 1e-5, gelu=False)
    close32(y, c["y"])
    c2 = golden.case("c2_ln_f32_5x1023")
    yg = O.ref_g2_layernorm(c2["x"], c2["gamma"], c2["beta"], 1e-5, gelu=True)
    close32(yg, c2["y_gelu_tanh"])


def test_torch_composition_matches_oracle_on_fresh_seed():
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(9, 520, generator=g) * 2).to(torch.bfloat16)
    res = torch.randn(9, 520, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(520, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(520, generator=g)).to(torch.bfloat16)
    for kind in ("layernorm", "rmsnorm"):
        b = beta if kind == "layernorm" else None
        a = O.norm_forward(x, gamma, b, res, kind, 1e-5)
        t = O.torch_forward(x, gamma, b, res, kind, 1e-5)
        assert int(O.ulp_distance_16(a["y"], t["y"]).max()) <= 1
        assert torch.equal(a["sum"].view(torch.int16), t["sum"].view(torch.int16))


def test_scaled_fp8_quantizers_match_torch_cast():
    """The two one-pass quantizers (caller-supplied scale, per-row scale) against torch's own
    e4m3 cast of the clamped product."""
    g = torch.Generator().manual_seed(77)
    y = torch.randn(33, 512, generator=g) * 3
    y[3] = 0
    y[5, 7] = 1e4  # saturates under the stale scale below
    q, amax = O.quant_fp8_delayed(y, 20.0)
    want = (y * 20.0).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(q, want)
    assert float(amax) == float(y.abs().max())
    q, scale, amax = O.quant_fp8_rowwise(y)
    rmax = y.abs().amax(-1)
    # IEEE fp32 division (via float64, which rounds to the same fp32); `448.0 / tensor` in
    # torch is a reciprocal and a multiply, i.e. two roundings
    assert torch.equal(scale, torch.where(rmax > 0, (448.0 / rmax.double()).float(), torch.ones_like(rmax)))
    want = (y * scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(q, want)
    assert float(scale[3]) == 1.0 and int(q[3].max()) == 0


def test_mxfp8_quantizer_matches_torch_composition():
    """Block-scaled quantizer against the same thing spelled with torch primitives
    (frexp for floor(log2), the float8 casts for the codes and the E8M0 byte)."""
    g = torch.Generator().manual_seed(78)
    y = torch.randn(9, 256, generator=g) * torch.logspace(-3, 3, 9)[:, None]
    y[2, 32:64] = 0
    y[4, 5] = 3e4
    q, e8 = O.quant_mxfp8(y)
    blocks = y.reshape(9, 8, 32)
    amax = blocks.abs().amax(-1)
    _, ex = torch.frexp(amax)                      # amax = m * 2^ex, m in [0.5, 1)
    want_e = torch.where(amax > 0, ex - 1 - 8 + 127, torch.zeros_like(ex)).clamp(min=0)
    assert torch.equal(e8.to(torch.int32), want_e.to(torch.int32))
    scale = torch.pow(2.0, want_e.double() - 127).float()
    if hasattr(torch, "float8_e8m0fnu"):
        assert torch.equal(scale[amax > 0].to(torch.float8_e8m0fnu).view(torch.uint8), e8[amax > 0])
    want_q = (blocks / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).reshape(9, 256)
    assert torch.equal(q, want_q)
    assert int(q[2, 32:64].max()) == 0 and int(e8[2, 1]) == 0
    # the largest element of every block lands in [256, 512) before saturation: top binade
    top = (blocks / scale[..., None]).abs().amax(-1)[amax > 0]
    assert bool(((top >= 256) & (top < 512)).all())


def test_philox_known_answers_and_keep_rate():
    """The generator behind the fused dropout: Philox4x32-10 against the known-answer vectors
    published with the algorithm (Random123 kat_vectors: zero, all-ones and pi-digits inputs),
    and the keep rate of the mask derived from it."""
    assert [hex(v) for v in O.philox4x32_10([0, 0, 0, 0], [0, 0])] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    assert [hex(v) for v in O.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2)] == \
        ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    assert [hex(v) for v in O.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0])] == \
        ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]
    n = 1 << 20
    for p in (0.0, 0.1, 0.5):
        bits = O.dropout_keep_bits(99, 7, p, n)
        kept = int(torch.tensor(np.unpackbits(bits.numpy())).sum())
        assert abs(kept / n - (1 - p)) < 4e-3
    assert not torch.equal(O.dropout_keep_bits(99, 7, 0.5, n), O.dropout_keep_bits(99, 8, 0.5, n))  # the offset matters
    assert not torch.equal(O.dropout_keep_bits(99, 7, 0.5, n), O.dropout_keep_bits(100, 7, 0.5, n))  # and the seed
    x = torch.arange(16, dtype=torch.float32) + 1
    bits = torch.tensor([0b10100101, 0xff], dtype=torch.uint8)
    out = O.dropout_apply(x, bits, 0.5)
    assert out.tolist() == [2, 0, 6, 0, 0, 12, 0, 16, 18, 20, 22, 24, 26, 28, 30, 32]
