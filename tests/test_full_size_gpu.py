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


def test_full_fp8_softmax_configuration_sampled_parity(G):
    """B=1024, H=4, D=128, L ~ U[128, 2048], FP8 e4m3 inputs with per-128-token-block scales, softmax, scale
    1/sqrt(D), bf16 output: the whole batch in one launch; the three shortest sequences, a median and the longest
    one against the oracle on their DE-QUANTISED inputs, at the stated FP8 bound (atol 5e-2, rtol 1e-1, at most
    1 % of the elements outside)."""
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload

    w = make_workload("c4_fp8_softmax")
    t = make_tensors(w, torch.device("cuda"), seed=9, dtype=torch.float32)
    qo = t["q_offsets"]
    q8, sq, qb = G.quantize_fp8_blockwise(t["q"], qo)
    k8, sk, kb = G.quantize_fp8_blockwise(t["k"], qo)
    v8, sv, vb = G.quantize_fp8_blockwise(t["v"], qo)
    mx = int(w.q_lens.max())
    o = G.generalized_dot_product_attention_fp8(q8, k8, v8, sq, sk, sv, qb, kb, qo, qo, mx, mx, qk_scale=w.qk_scale,
                                                activation="softmax")
    torch.cuda.synchronize()
    assert G.kernel_status() == 0 and o.dtype == torch.bfloat16 and torch.isfinite(o.float()).all()
    # repeatability: the forward has no atomics
    o2 = G.generalized_dot_product_attention_fp8(q8, k8, v8, sq, sk, sv, qb, kb, qo, qo, mx, mx, qk_scale=w.qk_scale,
                                                 activation="softmax")
    assert torch.equal(o, o2)
    off, boff = qo.cpu(), qb.cpu()

    def deq(x8, s, b):
        r0, r1, b0 = int(off[b]), int(off[b + 1]), int(boff[b])
        rows = x8[r0:r1].float().cpu()
        blk = torch.arange(r1 - r0) // 128 + b0
        return rows * s.cpu()[blk].unsqueeze(-1)

    order = np.argsort(w.q_lens)
    worst = 0.0
    for b in [int(i) for i in order[:3]] + [int(order[len(order) // 2]), int(order[-1])]:
        n = int(w.q_lens[b])
        one = torch.tensor([0, n])
        ref = orc.gdpa_forward(deq(q8, sq, b), deq(k8, sk, b), deq(v8, sv, b), one, one, "softmax", w.qk_scale)
        got = o[int(off[b]):int(off[b + 1])].float().cpu()
        err = (got - ref).abs()
        outside = (err > 5e-2 + 1e-1 * ref.abs()).float().mean().item()
        worst = max(worst, float(err.max()))
        assert outside <= 0.01, f"sequence {b} (length {n}): {outside:.4f} of the elements outside the FP8 bound"
    assert worst < 0.25  # softmax outputs are averages of N(0,1) values: errors stay far below one


def test_full_zipf_shard_sampled_parity(G):
    """One token-balanced shard (1/8) of the B=8192 Zipf(1.2) configuration (H=4, D=128, lengths 32 ... 8192,
    GELU-tanh, scale 1/8192), forward and backward in one launch each, as a rank of the 8-GPU split runs it; the three
    shortest sequences, a median one and one at the 8 192-token cap against the fp32 oracle."""
    from ads_model_kernel_library_b200.gdpa.sharding import plan_token_balanced_shards
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload

    w = make_workload("c5_zipf_sharded")
    s, e = plan_token_balanced_shards(w.q_lens, w.kv_lens, 8)[0]
    t = make_tensors(w, torch.device("cuda"), seed=10, with_grad_out=True, seq_range=(s, e))
    lens = w.q_lens[s:e]
    mq = int(lens.max())
    assert mq == 8192
    q, k, v = (t[n].requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, t["q_offsets"], t["kv_offsets"], mq, mq, qk_scale=w.qk_scale,
                                            activation=w.activation)
    o.backward(t["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    for x in (o, q.grad, k.grad, v.grad):
        assert torch.isfinite(x.float()).all()
    order = np.argsort(lens, kind="stable")
    sample = [int(i) for i in order[:3]] + [int(order[len(order) // 2]), int(order[-1])]

    class W:  # the fields _sample_check reads
        qk_scale = w.qk_scale

    tt = {n: t[n].detach() for n in ("q", "k", "v", "do", "q_offsets", "kv_offsets")}
    _sample_check(G, W, tt, o.detach(), (q.grad, k.grad, v.grad), w.activation, sample)
