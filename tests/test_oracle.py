"""The CPU oracle against the golden vectors produced by the reference's own Python code
(tests/golden/make_golden.py), and internal consistency of the oracle (autograd route against the
closed-form derivative tables)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))


def test_activation_ids_match_reference_table():
    ids = json.load(open(os.path.join(HERE, "golden", "activation_ids.json")))
    assert ids == orc.ACTIVATION_IDS


def test_softmax_matches_reference_cpu_kernel(golden):
    t = lambda n: torch.from_numpy(golden[n])
    out = orc.gdpa_forward(t("softmax_q"), t("softmax_k"), t("softmax_v"), t("softmax_qo"), t("softmax_ko"),
                           activation="softmax", qk_scale=None)
    torch.testing.assert_close(out, t("softmax_out"), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("act", list(orc.ACTIVATION_IDS))
def test_activations_match_reference_eager_helper(golden, act):
    t = lambda n: torch.from_numpy(golden[n])
    out = orc.gdpa_forward(t("eager_q"), t("eager_k"), t("eager_v"), t("eager_off"), t("eager_off"),
                           activation=act, qk_scale=None)
    torch.testing.assert_close(out, t(f"eager_out_{act}"), atol=1e-5, rtol=1e-5)


def test_scale_is_applied_after_the_activation(golden):
    t = lambda n: torch.from_numpy(golden[n])
    base = t("eager_out_gelu_approx")
    out = orc.gdpa_forward(t("eager_q"), t("eager_k"), t("eager_v"), t("eager_off"), t("eager_off"),
                           activation="gelu_approx", qk_scale=0.125)
    torch.testing.assert_close(out, base * 0.125, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("act", ["raw", "gelu", "gelu_approx", "leaky_relu", "relu", "silu", "hardswish", "relu_square"])
def test_autograd_matches_closed_form_derivatives(act):
    rng = np.random.default_rng(7)
    lq, lk = rng.integers(1, 30, 4), rng.integers(1, 30, 4)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]))
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    g = torch.Generator().manual_seed(7)
    q = torch.randn(int(qo[-1]), 2, 8, generator=g, dtype=torch.float64)
    k = torch.randn(int(ko[-1]), 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(int(ko[-1]), 2, 8, generator=g, dtype=torch.float64)
    do = torch.randn(int(qo[-1]), 2, 8, generator=g, dtype=torch.float64)
    _, dq, dk, dv = orc.gdpa_forward_backward(q, k, v, qo, ko, do, act, 0.3)
    dq2, dk2, dv2 = orc.gdpa_backward_formulas(q, k, v, qo, ko, do, act, 0.3)
    for a, b in ((dq, dq2), (dk, dk2), (dv, dv2)):
        torch.testing.assert_close(a, b, atol=2e-4, rtol=2e-4)


def test_empty_sequences_and_unknown_activation():
    qo = torch.tensor([0, 0, 3, 3])
    ko = torch.tensor([0, 2, 2, 5])
    q, k, v = torch.randn(3, 1, 4), torch.randn(5, 1, 4), torch.randn(5, 1, 4)
    out = orc.gdpa_forward(q, k, v, qo, ko, "relu", 1.0)
    assert torch.equal(out, torch.zeros_like(out))  # the only non-empty Q has an empty KV
    with pytest.raises(ValueError):
        orc.gdpa_forward(q, k, v, qo, ko, "tanh", 1.0)


def test_useful_flops_formula():
    assert orc.useful_flops([2, 3], [5, 7], 4, 128, "fwd") == 4 * 4 * 128 * 31
    assert orc.useful_flops([2, 3], [5, 7], 4, 128, "fwd_bwd") == 14 * 4 * 128 * 31


# Activations whose Triton implementation ran under Triton's interpreter when the fixtures were made
# (the others are written with inline PTX, which the interpreter cannot execute).
# fast_gelu_taylor_approx also ran, but the kernel evaluates it with a low-degree polynomial that is only
# meaningful for |S| < 1.5 (the fixture's scores are N(0, 16)), while the reference's eager table
# (get_pytorch_activation), which this library follows, defines it as tanh-GELU: it is not compared.
TRITON_ACTS = ["raw", "gelu_approx", "leaky_relu", "relu", "silu", "hardswish", "relu_square"]


@pytest.mark.parametrize("act", TRITON_ACTS)
def test_oracle_matches_reference_triton_kernels_forward_and_backward(golden, act):
    """O, dQ, dK, dV of the reference's own Triton forward / backward kernels (run on the CPU by the
    Triton interpreter, qk_scale = 0.25, Q and KV lengths differ): pins where the scale is applied and
    every gradient."""
    t = lambda n: torch.from_numpy(golden[n])
    scale = float(golden["triton_scale"])
    o, dq, dk, dv = orc.gdpa_forward_backward(t("triton_q"), t("triton_k"), t("triton_v"), t("triton_qo"), t("triton_ko"),
                                              t("triton_do"), act, scale)
    tol = 2e-5
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, t(f"triton_{act}_{name}"), atol=tol, rtol=tol)


def test_oracle_matches_reference_triton_kernels_grouped_query(golden):
    t = lambda n: torch.from_numpy(golden[n])
    o, dq, dk, dv = orc.gdpa_forward_backward(t("gqa_q"), t("gqa_k"), t("gqa_v"), t("triton_qo"), t("triton_ko"), t("gqa_do"),
                                              "gelu_approx", float(golden["triton_scale"]))
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, t(f"gqa_{name}"), atol=2e-5, rtol=2e-5)


def test_oracle_matches_reference_triton_kernels_banded(golden):
    """window_size: pairs with |q - kv| > W are zeroed before the activation, forward and backward."""
    t = lambda n: torch.from_numpy(golden[n])
    o, dq, dk, dv = orc.gdpa_forward_backward(t("triton_q"), t("triton_k"), t("triton_v"), t("triton_qo"), t("triton_ko"),
                                              t("triton_do"), "gelu_approx", float(golden["triton_scale"]),
                                              window_size=int(golden["window_size"]))
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, t(f"window_{name}"), atol=2e-5, rtol=2e-5)


def test_oracle_matches_reference_triton_kernels_per_head_activations(golden):
    """ensemble_activation_list: head 0 relu, head 1 leaky_relu."""
    t = lambda n: torch.from_numpy(golden[n])
    names = {5: "relu", 4: "leaky_relu"}
    acts = [names[int(i)] for i in golden["ensemble_ids"]]
    scale = float(golden["triton_scale"])
    res = orc.forward_backward_of(
        lambda q, k, v: orc.gdpa_forward_ensemble(q, k, v, t("triton_qo"), t("triton_ko"), acts, scale),
        t("triton_q"), t("triton_k"), t("triton_v"), t("triton_do"))
    for name, got in zip(("o", "dq", "dk", "dv"), res):
        torch.testing.assert_close(got, t(f"ensemble_{name}"), atol=2e-5, rtol=2e-5)


def test_oracle_matches_reference_triton_kernels_broadcast_q(golden):
    """broadcast_q: one Q sequence for the whole batch, output [B * Lq, H, D], dQ summed over the batch."""
    t = lambda n: torch.from_numpy(golden[n])
    scale = float(golden["triton_scale"])
    res = orc.forward_backward_of(
        lambda q, k, v: orc.gdpa_forward_broadcast_q(q, k, v, t("triton_ko"), "gelu_approx", scale),
        t("bcast_q"), t("triton_k"), t("triton_v"), t("bcast_do"))
    for name, got in zip(("o", "dq", "dk", "dv"), res):
        torch.testing.assert_close(got, t(f"bcast_{name}"), atol=3e-5, rtol=3e-5)


def test_oracle_matches_reference_triton_kernels_start_end_offsets(golden):
    """use_start_end_offsets: [start, end] pairs per sequence, overlapping K / V ranges (dK / dV summed over the
    sequences that read a row), a Q row that no sequence owns."""
    t = lambda n: torch.from_numpy(golden[n])
    scale = float(golden["triton_scale"])
    qp, kp = golden["startend_q_pairs"], golden["startend_k_pairs"]
    assert kp[2] < kp[1] and qp[3] < qp[4]  # the fixture really overlaps K / V and leaves a Q gap
    res = orc.forward_backward_of(
        lambda q, k, v: orc.gdpa_forward_start_end(q, k, v, qp, kp, "gelu_approx", scale),
        t("triton_q"), t("triton_k"), t("triton_v"), t("triton_do"))
    for name, got in zip(("o", "dq", "dk", "dv"), res):
        torch.testing.assert_close(got, t(f"startend_{name}"), atol=3e-5, rtol=3e-5)


def test_norm_pipeline_oracle_follows_the_reference_test_formulation():
    """LayerNorm(Q) -> GDPA -> + ln_q -> RMSNorm, written as the reference's megakernel test writes it
    (gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:110-127) with torch's functional norms."""
    torch.manual_seed(0)
    T, H, D = 40, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, H, D), torch.randn(T, H, D)
    off = torch.tensor([0, 17, 40])
    ln_q = torch.nn.functional.layer_norm(q.view(T, -1), (H * D,), eps=1e-5).view_as(q)
    g = orc.gdpa_forward(ln_q, k, v, off, off, "fast_gelu", None)
    ref = torch.nn.functional.rms_norm((g + ln_q).view(T, -1), (H * D,), eps=1e-5).view_as(g)
    out = orc.gdpa_with_norms(q, k, v, off, off, "fast_gelu", None, fused_layernorm=True, fused_q_residual_add=True,
                              fused_rms_norm=True)
    torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-6)
    ref1 = torch.nn.functional.rms_norm(orc.gdpa_forward(q, k, v, off, off, "fast_gelu", None).view(T, -1), (H * D,),
                                        eps=1e-5).view_as(g)
    torch.testing.assert_close(orc.gdpa_with_norms(q, k, v, off, off, "fast_gelu", None, fused_rms_norm=True), ref1,
                               atol=1e-6, rtol=1e-6)


def test_fp8_block_format_restatement_properties():
    """The CPU restatement of the FP8 input format: one scale per (128-token block of a sequence, head), codes
    within e4m3's half-ulp of x / scale, the block maximum mapped to +-448."""
    lens = [130, 0, 5, 256]
    off = torch.tensor([0, 130, 130, 135, 391])
    g = torch.Generator().manual_seed(3)
    x = torch.randn(391, 2, 16, generator=g) * 3
    x8, sc, bo = orc.quantize_fp8_blockwise(x, off)
    assert bo.tolist() == [0, 2, 2, 3, 5] and sc.shape == (5, 2)
    # block 1 of sequence 0 holds rows 128, 129 only
    torch.testing.assert_close(sc[1], x[128:130].abs().amax(dim=(0, 2)) / 448.0)
    deq = x8.float()
    for b, (s, e) in enumerate(zip(off[:-1].tolist(), off[1:].tolist())):
        for j, r0 in enumerate(range(s, e, 128)):
            r1 = min(r0 + 128, e)
            y = x[r0:r1] / sc[bo[b] + j].view(1, 2, 1)
            assert float((deq[r0:r1] - y).abs().max()) <= 16.0 + 1e-3  # half an ulp at the top binade of e4m3
            assert float(deq[r0:r1].abs().max()) == 448.0
            rel = ((deq[r0:r1] - y).abs() / y.abs().clamp_min(2.0 ** -6))
            assert float(rel.max()) <= 2.0 ** -4 + 1e-6


def test_mxfp8_scale_code_known_answers():
    """e8m0 codes by the round-up rule of the reference's P quantisation (gdpa/src/activation_utils.py:444-517):
    exponent field of amax / 448, plus one when the mantissa is not zero."""
    amax = torch.tensor([448.0, 449.0, 1.0, 0.0, 224.0, 448.0 * 2.0 ** -20, 448.0 * 2.0 ** 10 * 1.5])
    assert orc.mx_e8m0_codes(amax).tolist() == [127, 128, 119, 0, 126, 107, 138]
    # the scaled block maximum never exceeds e4m3's largest value
    g = torch.Generator().manual_seed(11)
    a = torch.rand(4096, generator=g) * torch.pow(2.0, torch.randint(-40, 40, (4096,), generator=g).float())
    scaled = a.double() * torch.pow(2.0, (127 - orc.mx_e8m0_codes(a)).double())
    assert float(scaled.max()) <= 448.0 * (1 + 2.0 ** -22) and float(scaled.min()) > 224.0 * (1 - 2.0 ** -22)


def test_mxfp8_scale_atom_layout():
    """One 512-byte atom holds 128 rows x 4 scales, byte 16 * (row % 32) + 4 * (row / 32) + k: every byte once."""
    rows = torch.arange(128).view(128, 1)
    ks = torch.arange(4).view(1, 4)
    idx = orc.mx_scale_atom_byte(rows, ks).reshape(-1)
    assert sorted(idx.tolist()) == list(range(512))
    assert int(orc.mx_scale_atom_byte(torch.tensor(33), torch.tensor(2))) == 16 + 4 + 2


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_mxfp8_restatement_round_trip(axis, D):
    """Quantise -> de-quantise: every element within half an e4m3 ulp of its block's scale, scale rows padded
    per sequence to 128, scale bytes of rows that do not exist zero, cu_seqlens_sf 128-aligned prefix sums."""
    off = torch.tensor([0, 130, 130, 135, 391])
    g = torch.Generator().manual_seed(5)
    x = torch.randn(391, 2, D, generator=g) * torch.exp(2 * torch.randn(391, 2, 1, generator=g))
    x8, sf, cu = orc.quantize_mxfp8(x, off, axis)
    assert cu.tolist() == [0, 256, 256, 384, 640] and cu.dtype == torch.int32
    d_atoms = (D + 127) // 128
    assert sf.numel() == 2 * d_atoms * 5 * 512
    y = orc.dequantize_mxfp8(x8, sf, off, axis)
    # block maxima: along D (axis 0) per 32 elements of a row; along the tokens (axis 1) per 32 rows of a sequence
    if axis == 0:
        amax = x.reshape(391, 2, D // 32, 32).abs().amax(-1, keepdim=True).expand(-1, -1, -1, 32).reshape(391, 2, D)
    else:
        amax = torch.zeros_like(x)
        for s, e in zip(off[:-1].tolist(), off[1:].tolist()):
            for r0 in range(s, e, 32):
                r1 = min(r0 + 32, e)
                amax[r0:r1] = x[r0:r1].abs().amax(0, keepdim=True)
    # the block maximum lands in [224, 448], where an e4m3 ulp is 32: error <= 16 / 224 of the block maximum
    assert float(((y - x).abs() / amax.clamp_min(1e-30)).max()) <= 16.0 / 224.0 + 1e-6
    rel = (y - x).abs() / x.abs().clamp_min(1e-30)
    big = x.abs() >= amax * 2.0 ** -6  # normal range of the scaled e4m3 code
    assert float(rel[big].max()) <= 2.0 ** -4 + 1e-6
    # a larger layout (upper bound of blocks) holds the same scales at a different head stride
    x8b, sfb, _ = orc.quantize_mxfp8(x, off, axis, sf_blocks=8)
    assert torch.equal(x8b.view(torch.uint8), x8.view(torch.uint8))
    torch.testing.assert_close(orc.dequantize_mxfp8(x8b, sfb, off, axis, sf_blocks=8), y, atol=0, rtol=0)
    # rows 130..255 of sequence 0's second block do not exist: their scale bytes stay zero (axis 0)
    if axis == 0:
        atom = sf[(0 * 5 + 1) * d_atoms * 512:(0 * 5 + 1) * d_atoms * 512 + 512].view(32, 4, 4)
        assert int(atom[2:, 0].sum()) == 0 and int(atom[:, 1:].sum()) == 0 and int(atom[:2, 0, :min(4, D // 32)].min()) > 0


def _bf16(golden, name):
    return torch.from_numpy(golden[name]).view(torch.bfloat16)


def test_norm_pipeline_oracle_pinned_by_the_reference_tests_own_expected_values(golden):
    """The expected tensors of the reference's two GDPA-plus-norm tests (gdpa_megakernel/tests/
    test_tlx_gdpa_megakernel.py:50-91 and :93-145), computed by the reference's own statements (see make_golden.py),
    against `gdpa_with_norms` on the same bf16 inputs.  The reference rounds its intermediate results to bf16 (the
    GDPA output, the normalised Q); the oracle keeps fp32 except for the normalised Q, so the two agree to bf16
    rounding of values of order one."""
    q, k, v = (_bf16(golden, f"norms_{n}_bf16_bits") for n in ("q", "k", "v"))
    off = torch.from_numpy(golden["norms_offsets"])
    assert q.shape == (256, 2, 128) and off.tolist() == [0, 128, 256]
    rms = orc.gdpa_with_norms(q, k, v, off, off, "fast_gelu", None, fused_rms_norm=True)
    torch.testing.assert_close(rms, _bf16(golden, "norms_rms_ref_bf16_bits").float(), atol=2e-2, rtol=2e-2)
    both = orc.gdpa_with_norms(q, k, v, off, off, "fast_gelu", None, fused_layernorm=True, fused_q_residual_add=True,
                               fused_rms_norm=True, round_dtype=torch.bfloat16)
    torch.testing.assert_close(both, _bf16(golden, "norms_ln_rms_ref_bf16_bits").float(), atol=2e-2, rtol=2e-2)
    # mean absolute difference: far below one bf16 ulp of the values (order one), i.e. the same function
    assert float((both - _bf16(golden, "norms_ln_rms_ref_bf16_bits").float()).abs().mean()) < 3e-3
    assert float((rms - _bf16(golden, "norms_rms_ref_bf16_bits").float()).abs().mean()) < 3e-3
