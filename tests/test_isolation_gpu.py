"""A sequence's result depends on that sequence's rows only.

The kernels fetch 128-row tiles, so the last tile of a sequence also holds the first rows of the next sequence in
the packed tensors.  The reference's per-sequence block loads read such rows as zero
(gdpa/triton/triton_generalized_dot_product_attention.py:270, :317, :1575-1600), so nothing a neighbour holds -- Inf and
NaN included -- can reach another sequence's output or gradients.  These tests poison one sequence of a batch and
require every other sequence's O, dQ, dK, dV to be bit-for-bit what they are with clean inputs."""
import numpy as np
import pytest
import torch

from tests._util import assert_close, jagged_inputs, oracle_forward_backward

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


def _run(G, dev, lq, lk, act, scale):
    q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], int(max(lq)), int(max(lk)), qk_scale=scale,
                                            activation=act)
    o.backward(dev["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    return o.detach(), q.grad, k.grad, v.grad


def _rows_outside(t, off, b):
    s, e = int(off[b]), int(off[b + 1])
    return torch.cat([t[:s], t[e:]])


# ragged lengths on both sides of the poisoned sequence: tails of 1 ... 127 rows, tails that end exactly on a K slice
# of 16, single-tile and multi-tile sequences, Q and KV lengths that differ
LQ = [70, 200, 129, 1, 300, 256, 17, 140]
LK = [200, 77, 260, 9, 131, 128, 33, 500]


@pytest.mark.parametrize("act", ["gelu_approx", "silu", "relu", "softmax"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("poison", [float("inf"), float("nan")])
def test_non_finite_neighbour_does_not_leak(G, act, D, poison):
    cpu, dev = jagged_inputs(LQ, LK, 2, D, seed=61, std=0.5)
    scale = 1.0 / 16
    clean = _run(G, dev, LQ, LK, act, scale)
    for b in (1, 4, 6):
        bad = {n: t.clone() for n, t in dev.items()}
        qs, qe = int(cpu["qo"][b]), int(cpu["qo"][b + 1])
        ks, ke = int(cpu["ko"][b]), int(cpu["ko"][b + 1])
        bad["q"][qs:qe] = poison
        bad["do"][qs:qe] = poison
        bad["k"][ks:ke] = poison
        bad["v"][ks:ke] = poison
        got = _run(G, bad, LQ, LK, act, scale)
        for name, g, c, off in (("O", got[0], clean[0], cpu["qo"]), ("dQ", got[1], clean[1], cpu["qo"]),
                                ("dK", got[2], clean[2], cpu["ko"]), ("dV", got[3], clean[3], cpu["ko"])):
            a, e = _rows_outside(g, off, b), _rows_outside(c, off, b)
            assert torch.isfinite(a.float()).all(), f"{name}: non-finite values outside poisoned sequence {b}"
            if name == "dQ":  # an fp32 sum in a different order of atomic additions, rounded once
                assert_close(a, e.float(), f"{name} outside poisoned sequence {b}", atol=1e-3, rtol=1e-2)
            else:
                assert torch.equal(a, e), f"{name} of other sequences changed when sequence {b} was poisoned"


def test_non_finite_rows_beyond_the_batch_do_not_leak(G):
    """Rows of the packed tensors that no sequence owns (a gap after the last sequence) may hold anything."""
    lq, lk = [100, 37], [64, 200]
    cpu, dev = jagged_inputs(lq + [60], lk + [90], 2, 128, seed=62, std=0.5)
    for n in ("qo", "ko"):  # drop the last sequence from the offsets: its rows stay in the tensors, unowned
        dev[n] = dev[n][:-1].contiguous()
        cpu[n] = cpu[n][:-1].contiguous()
    clean = _run(G, dev, lq, lk, "gelu_approx", 0.05)
    bad = {n: t.clone() for n, t in dev.items()}
    bad["q"][137:] = float("nan")
    bad["do"][137:] = float("inf")
    bad["k"][264:] = float("nan")
    bad["v"][264:] = float("inf")
    got = _run(G, bad, lq, lk, "gelu_approx", 0.05)
    for name, g, c, rows in (("O", got[0], clean[0], 137), ("dQ", got[1], clean[1], 137), ("dK", got[2], clean[2], 264),
                             ("dV", got[3], clean[3], 264)):
        assert torch.isfinite(g[:rows].float()).all(), name
        if name == "dQ":
            assert_close(g[:rows], c[:rows].float(), name, atol=1e-3, rtol=1e-2)
        else:
            assert torch.equal(g[:rows], c[:rows]), name
    ro, rdq, rdk, rdv = oracle_forward_backward({n: (t[:137] if n in ("q", "do") else t[:264] if n in ("k", "v") else t)
                                                  for n, t in cpu.items()}, "gelu_approx", 0.05)
    assert_close(got[0][:137], ro, "O")
    assert_close(got[1][:137], rdq, "dQ")
    assert_close(got[2][:264], rdk, "dK")
    assert_close(got[3][:264], rdv, "dV")


def test_fp8_non_finite_neighbour_scales_do_not_leak(G):
    """FP8 forward: e4m3 has no Inf, but a NaN code (0x7f) in a neighbour's V rows must not reach this sequence."""
    lens = [200, 77, 260]
    off = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(63)
    x = [torch.randn(int(off[-1]), 2, 128, generator=g, device="cuda") for _ in range(3)]
    q8, sq, qb = G.quantize_fp8_blockwise(x[0], off)
    k8, sk, kb = G.quantize_fp8_blockwise(x[1], off)
    v8, sv, vb = G.quantize_fp8_blockwise(x[2], off)

    def run(k8_, v8_):
        o = G.generalized_dot_product_attention_fp8(q8, k8_, v8_, sq, sk, sv, qb, kb, off, off, 260, 260, qk_scale=0.09,
                                                    activation="softmax")
        torch.cuda.synchronize()
        assert G.kernel_status() == 0
        return o

    clean = run(k8, v8)
    k_bad, v_bad = k8.clone(), v8.clone()
    k_bad.view(torch.uint8)[200:277] = 0x7F
    v_bad.view(torch.uint8)[200:277] = 0x7F
    got = run(k_bad, v_bad)
    assert torch.isfinite(got[:200].float()).all() and torch.isfinite(got[277:].float()).all()
    assert torch.equal(got[:200], clean[:200]) and torch.equal(got[277:], clean[277:])
