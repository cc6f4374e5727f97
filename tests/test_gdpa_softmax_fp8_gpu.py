"""GPU parity of the softmax forward (bf16) and of the low-precision forward (FP8 e4m3 inputs with
per-128-token-block fp32 scales, softmax, bf16 output) against the CPU oracle.

bf16: atol = rtol = 2e-2 against the fp32 oracle on the bf16-rounded inputs.
FP8: the oracle runs on the DE-QUANTISED inputs; the stated looser bound is atol = 5e-2, rtol = 1e-1
with at most 1 % of the elements outside (P is re-quantised to e4m3 inside the kernel)."""
import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc
from tests._util import assert_close, jagged_inputs

pytestmark = pytest.mark.gpu

FP8_ATOL, FP8_RTOL, FP8_MAX_OUTSIDE = 5e-2, 1e-1, 0.01


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("scale", [None, 0.125])
def test_softmax_forward_matches_oracle(G, D, scale):
    lq, lk = [1, 70, 300, 129, 256, 513], [5, 200, 131, 260, 1000, 77]
    cpu, dev = jagged_inputs(lq, lk, 2, D, seed=31, std=0.7)
    o = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], max(lq), max(lk),
                                            qk_scale=scale, activation="softmax")
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ref = orc.gdpa_forward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"], "softmax", scale)
    assert_close(o, ref, "O[softmax]")


def test_softmax_running_maximum_is_rescaled(G):
    """Keys whose norm grows along the sequence make the row maximum jump from tile to tile, which
    exercises the rescaling of the O accumulator."""
    lq, lk = [200, 384], [1500, 2048]
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=32, std=0.5)
    for name in ("k",):
        ramp = torch.cat([torch.linspace(0.2, 3.0, n) for n in lk]).view(-1, 1, 1)
        cpu[name] = (cpu[name].float() * ramp).to(torch.bfloat16)
        dev[name] = cpu[name].cuda()
    o = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], max(lq), max(lk),
                                            qk_scale=1.0, activation="softmax")
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ref = orc.gdpa_forward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"], "softmax", 1.0)
    assert_close(o, ref, "O[softmax, growing keys]")


@pytest.mark.parametrize("D", [64, 128])
def test_softmax_backward_matches_oracle(G, D):
    """The trainable softmax variant: dQ, dK, dV against autograd over the fp32 oracle."""
    lq, lk = [1, 70, 300, 129, 256], [5, 200, 131, 260, 600]
    cpu, dev = jagged_inputs(lq, lk, 2, D, seed=33, std=0.5)
    scale = 0.125
    q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=scale,
                                            activation="softmax")
    o.backward(dev["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"],
                                                  cpu["do"].float(), "softmax", scale)
    assert_close(o, ro, "O[softmax]")
    assert_close(q.grad, rdq, "dQ[softmax]")
    assert_close(k.grad, rdk, "dK[softmax]")
    assert_close(v.grad, rdv, "dV[softmax]")


def test_softmax_backward_with_growing_keys_and_empty_sequences(G):
    lq, lk = [200, 0, 384, 17], [1500, 40, 1024, 0]
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=34, std=0.5)
    ramp = torch.cat([torch.linspace(0.2, 2.0, n) for n in lk if n > 0]).view(-1, 1, 1)
    cpu["k"] = (cpu["k"].float() * ramp).to(torch.bfloat16)
    dev["k"] = cpu["k"].cuda()
    q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=0.5,
                                            activation="softmax")
    o.backward(dev["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"],
                                                  cpu["do"].float(), "softmax", 0.5)
    # Growing keys make the row maximum jump from tile to tile (the forward rescales its accumulator) and
    # the softmax peaked; dS = P (dP - dPsum) then subtracts nearly equal numbers, with dPsum built from
    # the bf16-rounded O, so the absolute tolerance follows the scale of each tensor (2e-2 of its root
    # mean square, at least 2e-2); the relative one stays 2e-2.
    for a, b, n in ((o, ro, "O"), (q.grad, rdq, "dQ"), (k.grad, rdk, "dK"), (v.grad, rdv, "dV")):
        rms = float(b.float().pow(2).mean().sqrt())
        assert_close(a, b, n + "[softmax]", atol=2e-2 * max(1.0, rms), rtol=2e-2)


def _fp8_case(G, lq, lk, H, seed, scale, act="softmax"):
    rng = torch.Generator().manual_seed(seed)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]), dtype=torch.int64)
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]), dtype=torch.int64)
    q = torch.randn(int(qo[-1]), H, 128, generator=rng)
    k = torch.randn(int(ko[-1]), H, 128, generator=rng)
    v = torch.randn(int(ko[-1]), H, 128, generator=rng)
    q8, sq, qb = G.quantize_fp8_blockwise(q.cuda(), qo.cuda())
    k8, sk, kb = G.quantize_fp8_blockwise(k.cuda(), ko.cuda())
    v8, sv, vb = G.quantize_fp8_blockwise(v.cuda(), ko.cuda())
    o = G.generalized_dot_product_attention_fp8(q8, k8, v8, sq, sk, sv, qb, kb, qo.cuda(), ko.cuda(), int(max(lq)),
                                                int(max(lk)), qk_scale=scale, activation=act)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    assert o.dtype == torch.bfloat16

    def deq(x8, s, off):
        out = x8.float().cpu()
        lens = (off[1:] - off[:-1]).tolist()
        row = 0
        blk = 0
        s = s.cpu()
        for n in lens:
            for b0 in range(0, n, 128):
                out[row + b0:row + min(b0 + 128, n)] *= s[blk].view(1, H, 1)
                blk += 1
            row += n
        return out

    ref = orc.gdpa_forward(deq(q8, sq, qo), deq(k8, sk, ko), deq(v8, sv, ko), qo, ko, act, scale)
    got = o.float().cpu()
    assert torch.isfinite(got).all()
    err = (got - ref).abs()
    # softmax outputs are averages of V (order one); with an element-wise activation the output grows with the
    # scores and the sequence length, and so does the quantisation noise of P: the absolute part of the bound is
    # taken relative to the RMS of the reference there
    atol = FP8_ATOL if act == "softmax" else FP8_ATOL * max(1.0, float(ref.pow(2).mean().sqrt()))
    outside = (err > atol + FP8_RTOL * ref.abs()).float().mean().item()
    assert outside <= FP8_MAX_OUTSIDE, f"{outside:.4f} of the elements outside atol={atol} rtol={FP8_RTOL}; max err {err.max():.4g}"
    return float(err.max()), outside


def test_fp8_softmax_forward_within_stated_bound(G):
    _fp8_case(G, [128, 300, 77, 1, 640], [128, 515, 260, 9, 1000], 2, 41, 1.0 / np.sqrt(128.0))


def test_fp8_reduced_config4(G):
    """Lengths U[128, 2048], H=4, D=128, softmax, scale 1/sqrt(D): a reduced batch of the FP8 config."""
    rng = np.random.default_rng(3)
    ln = rng.integers(128, 2049, 6)
    _fp8_case(G, ln, ln, 4, 42, 1.0 / np.sqrt(128.0))


@pytest.mark.parametrize("act", ["gelu_approx", "silu", "relu", "raw", "hardswish", "leaky_relu", "gelu"])
def test_fp8_elementwise_activations_within_stated_bound(G, act):
    """FP8 operands with an element-wise activation: P is quantised to e4m3 after the activation (with the V-block
    scale folded in), the scale is applied to the fp32 accumulator.  Scores are N(0, 128) here, so |P| reaches ~50."""
    _fp8_case(G, [128, 300, 77, 1, 640], [128, 515, 260, 9, 1000], 2, 43, 1.0 / 64, act=act)


def test_fp8_rejects_other_head_dims(G):
    qo = torch.tensor([0, 16], device="cuda")
    x = torch.zeros(16, 1, 64, device="cuda")
    x8, s, b = G.quantize_fp8_blockwise(x, qo)
    with pytest.raises((RuntimeError, NotImplementedError)):
        G.generalized_dot_product_attention_fp8(x8, x8, x8, s, s, s, b, b, qo, qo, 16, 16, activation="gelu_approx")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("off_dtype", [torch.int64, torch.int32])
def test_fp8_block_quantiser_is_bit_exact_against_its_cpu_restatement(G, dtype, off_dtype):
    """Byte work: the e4m3 codes, the scales and the block offsets must equal the CPU restatement bit for bit
    (ragged lengths, an empty sequence, a length-1 sequence, zeros, values that saturate the block maximum)."""
    lens = [128, 300, 0, 77, 1, 640, 129]
    off = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=off_dtype)
    g = torch.Generator().manual_seed(77)
    x = (torch.randn(int(off[-1]), 3, 128, generator=g) * torch.logspace(-3, 2, 3).view(1, 3, 1)).to(dtype)
    x[5:9] = 0
    x8, sc, bo = G.quantize_fp8_blockwise(x.cuda(), off.cuda())
    torch.cuda.synchronize()
    r8, rsc, rbo = orc.quantize_fp8_blockwise(x, off)
    nb = int(rbo[-1])
    assert torch.equal(bo.cpu(), rbo)
    assert torch.equal(sc.cpu()[:nb], rsc) and torch.count_nonzero(sc.cpu()[nb:]) == 0
    assert torch.equal(x8.cpu().view(torch.uint8), r8.view(torch.uint8))
