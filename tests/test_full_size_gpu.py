"""GPU tests at the full size of the benchmark configurations: the operator runs on the whole batch (one launch,
the schedule and the persistent grid of the benchmark), and is checked (a) against the CPU oracle on a sample of
its sequences, whose rows are cut out of the full-size result, and (b) through size-independent properties."""
import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc
from tests._util import ATOL, RTOL, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


def _sample_check(G, w, t, o, grads, act, sample):
    """Oracle on the sequences `sample` alone (sequences are independent) against their rows of the full run."""
    qo, ko = t["q_offsets"].cpu(), t["kv_offsets"].cpu()
    for b in sample:
        qs, qe, ks, ke = int(qo[b]), int(qo[b + 1]), int(ko[b]), int(ko[b + 1])
        q, k, v = (t[n][s:e].float().cpu() for n, s, e in (("q", qs, qe), ("k", ks, ke), ("v", ks, ke)))
        off_q, off_k = torch.tensor([0, qe - qs]), torch.tensor([0, ke - ks])
        if grads is None:
            ro = orc.gdpa_forward(q, k, v, off_q, off_k, act, w.qk_scale)
            assert_close(o[qs:qe], ro, f"O of sequence {b}")
            continue
        ro, rdq, rdk, rdv = orc.gdpa_forward_backward(q, k, v, off_q, off_k, t["do"][qs:qe].float().cpu(), act, w.qk_scale)
        dq, dk, dv = grads
        for got, want, name in ((o[qs:qe], ro, "O"), (dq[qs:qe], rdq, "dQ"), (dk[ks:ke], rdk, "dK"), (dv[ks:ke], rdv, "dV")):
            assert_close(got, want, f"{name} of sequence {b}", atol=ATOL, rtol=RTOL)


def test_full_fwd_bwd_configuration_sampled_parity_and_properties(G):
    """B=512, H=8, D=128, L ~ U[512, 4096], GELU-tanh, forward and backward on 1.19 M tokens."""
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload

    w = make_workload("c3_fwd_bwd_gelu_uniform")
    t = make_tensors(w, torch.device("cuda"), seed=7, with_grad_out=True)
    mq = int(w.q_lens.max())

    def run(v, do):
        q, k, vv = t["q"].clone().requires_grad_(True), t["k"].clone().requires_grad_(True), v.clone().requires_grad_(True)
        o = G.generalized_dot_product_attention(q, k, vv, t["q_offsets"], t["kv_offsets"], mq, mq, qk_scale=w.qk_scale,
                                                activation=w.activation)
        o.backward(do)
        return o.detach(), q.grad, k.grad, vv.grad

    o, dq, dk, dv = run(t["v"], t["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    # (a) the four shortest sequences and one of the longest against the oracle
    order = np.argsort(w.q_lens)
    _sample_check(G, w, t, o, (dq, dk, dv), w.activation, [int(i) for i in order[:4]] + [int(order[-1])])
    # (b) bitwise repeatability of O, dK, dV (dQ is an fp32 atomic sum rounded once: equal up to that rounding)
    o2, dq2, dk2, dv2 = run(t["v"], t["do"])
    assert torch.equal(o, o2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert_close(dq2, dq, "dQ repeat", atol=1e-3, rtol=2e-2)
    # (c) linearity: dV is linear in dO (P does not depend on dO): dV(2 dO) == 2 dV(dO) exactly in bf16
    _, _, _, dv3 = run(t["v"], t["do"] * 2)
    assert torch.equal(dv3, dv * 2)
    # (d) every output is finite and rows of different sequences do not leak: zeroing the V of one sequence
    # changes the O rows of that sequence only
    b = int(order[len(order) // 2])
    ks, ke = int(t["kv_offsets"][b]), int(t["kv_offsets"][b + 1])
    qs, qe = int(t["q_offsets"][b]), int(t["q_offsets"][b + 1])
    v0 = t["v"].clone()
    v0[ks:ke] = 0
    with torch.no_grad():
        o0 = G.generalized_dot_product_attention(t["q"], t["k"], v0, t["q_offsets"], t["kv_offsets"], mq, mq,
                                                 qk_scale=w.qk_scale, activation=w.activation)
    assert torch.equal(o0[:qs], o[:qs]) and torch.equal(o0[qe:], o[qe:])
    assert torch.count_nonzero(o0[qs:qe]) == 0


def test_full_forward_configuration_sampled_parity(G):
    """B=1024, H=4, D=128, log-normal Q and KV lengths, SiLU forward."""
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload

    w = make_workload("c2_fwd_silu_lognormal")
    t = make_tensors(w, torch.device("cuda"), seed=8)
    with torch.no_grad():
        o = G.generalized_dot_product_attention(t["q"], t["k"], t["v"], t["q_offsets"], t["kv_offsets"], int(w.q_lens.max()),
                                                int(w.kv_lens.max()), qk_scale=w.qk_scale, activation=w.activation)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0 and torch.isfinite(o.float()).all()
    cost = w.q_lens * w.kv_lens
    order = np.argsort(cost)
    _sample_check(G, w, t, o, None, w.activation, [int(i) for i in order[:3]] + [int(order[len(order) // 2]), int(order[-1])])
