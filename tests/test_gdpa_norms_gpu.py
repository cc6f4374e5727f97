"""GPU parity tests of the GDPA-plus-norm pipeline (layer norm of Q, GDPA, Q residual, RMS norm, residual)
against the CPU oracle, with the tolerance of the reference's own test of that pipeline
(gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:91, :145): atol = rtol = 3e-2."""
import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc
from tests._util import assert_close, jagged_inputs

pytestmark = pytest.mark.gpu

NORM_ATOL = NORM_RTOL = 3e-2


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


@pytest.mark.parametrize("shape", [(37, 2, 128), (300, 8, 128), (129, 32, 128), (64, 2, 64), (5, 40, 128)])
def test_row_norm_kernels_against_torch(G, shape):
    """layernorm_rows / rmsnorm_rows alone, rows of 128 ... 5120 values (the row is kept in registers up to
    2048 values and re-read beyond)."""
    g = torch.Generator().manual_seed(5)
    T, H, D = shape
    x = (torch.randn(T, H, D, generator=g) * 2 + 0.3).to(torch.bfloat16)
    w = torch.randn(H * D, generator=g)
    b = torch.randn(H * D, generator=g)
    r = torch.randn(T, H, D, generator=g).to(torch.bfloat16)
    xf = x.float().reshape(T, H * D)
    ln = G.layernorm_rows(x.cuda(), w.cuda(), b.cuda())
    ref = torch.nn.functional.layer_norm(xf, (H * D,), w, b, 1e-5).reshape(T, H, D)
    assert_close(ln, ref, "layer norm", atol=2e-2, rtol=1e-2)
    ln0 = G.layernorm_rows(x.cuda())
    assert_close(ln0, torch.nn.functional.layer_norm(xf, (H * D,), None, None, 1e-5).reshape(T, H, D), "layer norm, plain",
                 atol=2e-2, rtol=1e-2)
    rms = G.rmsnorm_rows(x.cuda(), w.cuda(), r.cuda())
    ref = (xf * torch.rsqrt(xf.pow(2).mean(1, keepdim=True) + 1e-5) * w).reshape(T, H, D) + r.float()
    assert_close(rms, ref, "rms norm", atol=2e-2, rtol=1e-2)
    torch.cuda.synchronize()


def _run(G, cpu, dev, lq, lk, act, scale, **kw):
    dkw = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    out = G.gdpa_megakernel(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=scale,
                            activation=act, **dkw)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    okw = dict(kw)
    okw.pop("fused_residual_add", None)
    ref = orc.gdpa_with_norms(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"], act, scale,
                              round_dtype=torch.bfloat16, **okw)
    return out, ref


def test_fused_rmsnorm_dense_shape_of_the_reference_test(G):
    """batch 2 x 128 tokens, 2 heads of 128, fast_gelu, no scale: the case of the reference's own test."""
    cpu, dev = jagged_inputs([128, 128], [128, 128], 2, 128, seed=42, std=1.0)
    out, ref = _run(G, cpu, dev, [128, 128], [128, 128], "fast_gelu", None, fused_rms_norm=True)
    assert_close(out, ref, "rms(gdpa)", atol=NORM_ATOL, rtol=NORM_RTOL)


def test_fused_layernorm_q_residual_rmsnorm_dense_shape_of_the_reference_test(G):
    cpu, dev = jagged_inputs([128, 128], [128, 128], 2, 128, seed=42, std=1.0)
    out, ref = _run(G, cpu, dev, [128, 128], [128, 128], "fast_gelu", None, fused_layernorm=True,
                    fused_q_residual_add=True, fused_rms_norm=True)
    assert_close(out, ref, "rms(gdpa(ln q) + ln q)", atol=NORM_ATOL, rtol=NORM_RTOL)


@pytest.mark.parametrize("heads,D", [(2, 128), (8, 128), (4, 64)])
def test_jagged_pipeline_with_weights_and_generic_residual(G, heads, D):
    lq, lk = [300, 1, 129, 0, 257], [260, 70, 131, 50, 0]
    cpu, dev = jagged_inputs(lq, lk, heads, D, seed=8, std=0.7)
    g = torch.Generator().manual_seed(9)
    n = heads * D
    lw, lb, rw = 1 + 0.1 * torch.randn(n, generator=g), 0.1 * torch.randn(n, generator=g), 1 + 0.1 * torch.randn(n, generator=g)
    res = torch.randn(sum(lq), heads, D, generator=g).to(torch.bfloat16)
    out, ref = _run(G, cpu, dev, lq, lk, "gelu_approx", 1.0 / 64, fused_layernorm=True, layernorm_weight=lw,
                    layernorm_bias=lb, fused_q_residual_add=True, fused_rms_norm=True, rms_norm_weight=rw,
                    fused_residual_add=True, residual=res)
    assert_close(out, ref, "full pipeline", atol=NORM_ATOL, rtol=NORM_RTOL)
    # the pieces alone: Q residual without a norm, generic residual without a norm, nothing fused
    out, ref = _run(G, cpu, dev, lq, lk, "silu", 1.0 / 64, fused_q_residual_add=True)
    assert_close(out, ref, "gdpa + q", atol=NORM_ATOL, rtol=NORM_RTOL)
    out, ref = _run(G, cpu, dev, lq, lk, "relu", 1.0 / 64, fused_residual_add=True, residual=res)
    assert_close(out, ref, "gdpa + residual", atol=NORM_ATOL, rtol=NORM_RTOL)
    out, ref = _run(G, cpu, dev, lq, lk, "relu", 1.0 / 64)
    plain = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], max(lq), max(lk),
                                                qk_scale=1.0 / 64, activation="relu")
    assert torch.equal(out, plain)


def test_norm_pipeline_argument_errors(G):
    cpu, dev = jagged_inputs([10], [12], 2, 64, seed=1)
    args = (dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 10, 12)
    with pytest.raises(ValueError):
        G.gdpa_megakernel(*args, fused_layernorm=True)
    with pytest.raises(ValueError):
        G.gdpa_megakernel(*args, fused_residual_add=True)
    with pytest.raises(NotImplementedError):
        G.gdpa_megakernel(*args, is_causal=True)
    with pytest.raises(NotImplementedError):
        G.gdpa_megakernel(*args, activation="softmax", fused_rms_norm=True)


@pytest.mark.parametrize("case", ["rms", "ln_qres_rms", "all_weights", "qres_only", "residual_only"])
def test_norm_pipeline_backward_against_autograd_of_the_oracle(G, case):
    """Gradients of every input of the pipeline (Q, K, V, the norm weights / bias, the residual) against
    torch.autograd over the fp32 oracle."""
    lq, lk, heads, D = [300, 1, 129, 257], [260, 70, 131, 50], 2, 128
    cpu, dev = jagged_inputs(lq, lk, heads, D, seed=12, std=0.7)
    g = torch.Generator().manual_seed(13)
    n, T = heads * D, sum(lq)
    kw = {
        "rms": dict(fused_rms_norm=True),
        "ln_qres_rms": dict(fused_layernorm=True, fused_q_residual_add=True, fused_rms_norm=True),
        "all_weights": dict(fused_layernorm=True, layernorm_weight=1 + 0.1 * torch.randn(n, generator=g),
                            layernorm_bias=0.1 * torch.randn(n, generator=g), fused_q_residual_add=True, fused_rms_norm=True,
                            rms_norm_weight=1 + 0.1 * torch.randn(n, generator=g), fused_residual_add=True,
                            residual=torch.randn(T, heads, D, generator=g).to(torch.bfloat16)),
        "qres_only": dict(fused_q_residual_add=True),
        "residual_only": dict(fused_residual_add=True, residual=torch.randn(T, heads, D, generator=g).to(torch.bfloat16)),
    }[case]
    dout = (torch.randn(T, heads, D, generator=g) * 0.5).to(torch.bfloat16)
    scale, act = 1.0 / 64, "gelu_approx"
    # ---- GPU
    names = [k for k, v in kw.items() if isinstance(v, torch.Tensor)]
    dkw = {k: (v.cuda().requires_grad_(True) if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    q, k, v = (dev[x].clone().requires_grad_(True) for x in ("q", "k", "v"))
    out = G.gdpa_megakernel(q, k, v, dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=scale, activation=act, **dkw)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    # ---- oracle with autograd
    okw = {k: (v.float().clone().requires_grad_(True) if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    okw.pop("fused_residual_add", None)
    rq, rk, rv = (cpu[x].float().clone().requires_grad_(True) for x in ("q", "k", "v"))
    ref = orc.gdpa_with_norms(rq, rk, rv, cpu["qo"], cpu["ko"], act, scale, round_dtype=torch.bfloat16, **okw)
    ref.backward(dout.float())
    assert_close(out, ref, f"out[{case}]", atol=NORM_ATOL, rtol=NORM_RTOL)
    for name, got, want in (("dQ", q.grad, rq.grad), ("dK", k.grad, rk.grad), ("dV", v.grad, rv.grad)):
        assert_close(got, want, f"{name}[{case}]", atol=NORM_ATOL, rtol=NORM_RTOL)
    for name in names:
        want = okw[name].grad
        got = dkw[name].grad
        assert got is not None and got.shape == want.shape, name
        # weight / bias gradients are sums over all tokens: compare relative to their scale
        tol = NORM_ATOL * max(1.0, float(want.abs().max()))
        assert_close(got, want, f"d {name}[{case}]", atol=tol, rtol=NORM_RTOL)


def test_pipeline_reproduces_the_reference_tests_expected_values(G, golden):
    """The two cases of the reference's own GDPA-plus-norm test file on the reference's own inputs, against the
    expected tensors its statements produce (fixture generated by tests/golden/make_golden.py from the reference's
    source), at the reference's tolerance atol = rtol = 3e-2
    (gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:91, :145)."""
    bf = lambda n: torch.from_numpy(golden[n]).view(torch.bfloat16)
    q, k, v = (bf(f"norms_{n}_bf16_bits").cuda() for n in ("q", "k", "v"))
    off = torch.from_numpy(golden["norms_offsets"]).cuda()
    out = G.tlx_gdpa_megakernel(query=q, key=k, value=v, query_offset=off, key_offset=off, max_seq_len_q=128,
                                max_seq_len_kv=128, activation="fast_gelu", enable_tma=True, enable_ws=True,
                                fused_rms_norm=True)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    assert_close(out, bf("norms_rms_ref_bf16_bits").float(), "RMS norm after GDPA", atol=NORM_ATOL, rtol=NORM_RTOL)
    out = G.tlx_gdpa_megakernel(query=q, key=k, value=v, query_offset=off, key_offset=off, max_seq_len_q=128,
                                max_seq_len_kv=128, activation="fast_gelu", enable_tma=True, enable_ws=True,
                                fused_layernorm=True, fused_q_residual_add=True, fused_rms_norm=True)
    torch.cuda.synchronize()
    assert_close(out, bf("norms_ln_rms_ref_bf16_bits").float(), "layer norm, GDPA, residual, RMS norm", atol=NORM_ATOL,
                 rtol=NORM_RTOL)
