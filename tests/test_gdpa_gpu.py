"""GPU parity tests: the CUDA kernels (through the torch op, which calls the C ABI) against the CPU
oracle on the same seeded inputs.  bf16 kernels vs the fp32 oracle evaluated on the bf16-rounded
inputs: atol = rtol = 2e-2 on O, dQ, dK, dV."""
import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc
from tests._util import ATOL, RTOL, assert_close, jagged_inputs, oracle_forward, oracle_forward_backward

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


def run_fwd(G, dev, lq, lk, act, scale, max_q=None, max_kv=None):
    o = G.generalized_dot_product_attention(
        dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"],
        int(max(lq)) if max_q is None else max_q, int(max(lk)) if max_kv is None else max_kv,
        qk_scale=scale, activation=act)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    return o


def run_fwd_bwd(G, dev, lq, lk, act, scale):
    q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], int(max(lq)), int(max(lk)),
                                            qk_scale=scale, activation=act)
    o.backward(dev["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    return o, q.grad, k.grad, v.grad


ALL_ACTS = ["raw", "gelu", "gelu_approx", "fast_gelu", "leaky_relu", "relu", "fast_gelu_bf16", "silu", "fast_silu",
            "hardswish", "relu_square", "fast_gelu_taylor_approx"]


@pytest.mark.parametrize("act", ALL_ACTS)
@pytest.mark.parametrize("D", [64, 128])
def test_forward_backward_every_activation(G, act, D):
    lq, lk = [70, 300, 129], [200, 131, 260]
    # std 0.5 keeps |O| of order one for every activation (relu_square grows like S^2), which is the
    # range the absolute tolerance is meant for
    cpu, dev = jagged_inputs(lq, lk, 2, D, seed=3, std=0.5)
    scale = 1.0 / 64
    o, dq, dk, dv = run_fwd_bwd(G, dev, lq, lk, act, scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, act, scale)
    assert_close(o, ro, f"O[{act}]")
    assert_close(dq, rdq, f"dQ[{act}]")
    assert_close(dk, rdk, f"dK[{act}]")
    assert_close(dv, rdv, f"dV[{act}]")


EDGE_LENS = [1, 2, 15, 16, 17, 127, 128, 129, 255, 256, 257, 383, 385, 512, 513]


@pytest.mark.parametrize("D", [64, 128])
def test_edge_lengths_q_and_kv_differ(G, D):
    lq = EDGE_LENS
    lk = list(reversed(EDGE_LENS))
    cpu, dev = jagged_inputs(lq, lk, 3, D, seed=11, std=0.5)
    scale = 1.0 / 32
    o, dq, dk, dv = run_fwd_bwd(G, dev, lq, lk, "gelu_approx", scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "gelu_approx", scale)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)


def test_empty_sequences_and_single_sequence(G):
    # sequences with no queries, with no keys, with neither
    lq, lk = [0, 5, 130, 0, 64], [7, 0, 140, 0, 64]
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=5, std=0.5)
    o, dq, dk, dv = run_fwd_bwd(G, dev, lq, lk, "silu", 0.05)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "silu", 0.05)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)
    # B = 1
    cpu, dev = jagged_inputs([200], [300], 1, 64, seed=6, std=0.5)
    o, dq, dk, dv = run_fwd_bwd(G, dev, [200], [300], "relu", 0.1)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "relu", 0.1)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)


def test_int32_offsets_and_default_scale(G):
    lq, lk = [33, 257], [129, 64]
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=8, std=0.3, offset_dtype=torch.int32)
    o = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 257, 129,
                                            activation="gelu_approx")  # qk_scale=None -> 1.0
    ro = oracle_forward(cpu, "gelu_approx", None)
    assert_close(o, ro, "O")


def test_max_seq_len_clamps_lengths_like_the_reference(G):
    # The reference clamps each sequence to max_seq_len (qlen = min(qlen, N_CTX)); rows beyond are not written.
    lq, lk = [300, 100], [400, 90]
    cpu, dev = jagged_inputs(lq, lk, 1, 128, seed=9, std=0.5)
    o = run_fwd(G, dev, lq, lk, "relu", 0.1, max_q=200, max_kv=256)
    cpu2 = dict(cpu)
    # oracle on the clamped geometry
    from oracle import gdpa_oracle as orc
    q, k, v = cpu["q"].float(), cpu["k"].float(), cpu["v"].float()
    exp0 = orc.gdpa_forward(q[:200], k[:256], v[:256], torch.tensor([0, 200]), torch.tensor([0, 256]), "relu", 0.1)
    exp1 = orc.gdpa_forward(q[300:400], k[400:490], v[400:490], torch.tensor([0, 100]), torch.tensor([0, 90]), "relu", 0.1)
    assert_close(o[:200], exp0, "O[seq0 clamped]")
    assert_close(o[300:400], exp1, "O[seq1]")


def test_forward_is_bitwise_deterministic_and_backward_repeatable(G):
    lq, lk = [500, 77, 1000], [640, 300, 900]
    cpu, dev = jagged_inputs(lq, lk, 4, 128, seed=12, std=0.5)
    o1, dq1, dk1, dv1 = run_fwd_bwd(G, dev, lq, lk, "gelu_approx", 1e-3)
    o2, dq2, dk2, dv2 = run_fwd_bwd(G, dev, lq, lk, "gelu_approx", 1e-3)
    assert torch.equal(o1, o2)
    assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
    assert_close(dq1, dq2.float(), "dQ repeat", atol=1e-2, rtol=1e-2)  # fp32 reductions may reorder


def test_config1_shapes_fwd_bwd(G):
    """The reference's CPU-runnable configuration: B=8, H=2, D=64, lengths U[16,256], GELU-tanh,
    scale 1/max_kv, N(0,1) inputs."""
    from ads_model_kernel_library_b200.gdpa.workloads import make_workload

    w = make_workload("c1_cpu_small")
    cpu, dev = jagged_inputs(w.q_lens, w.kv_lens, w.heads, w.head_dim, seed=0)
    o, dq, dk, dv = run_fwd_bwd(G, dev, w.q_lens, w.kv_lens, w.activation, w.qk_scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, w.activation, w.qk_scale)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)


def test_reduced_config3_and_linearity_in_v_at_scale(G):
    """Self-attention lengths U[512,4096], H=8, D=128, N(0,0.5): a few sequences against the oracle,
    and a size-independent property on a larger batch: O is linear in V, so
    O(V1 + V2) == O(V1) + O(V2) up to bf16 rounding."""
    rng = np.random.default_rng(2)
    ln = rng.integers(512, 4097, 3)
    cpu, dev = jagged_inputs(ln, ln, 8, 128, seed=2, std=0.5)
    scale = 1.0 / int(ln.max())
    o, dq, dk, dv = run_fwd_bwd(G, dev, ln, ln, "gelu_approx", scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "gelu_approx", scale)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)
    ln = rng.integers(512, 4097, 64)
    _, dev = jagged_inputs(ln, ln, 8, 128, seed=3, std=0.5)
    v2 = torch.randn_like(dev["v"]) * 0.5
    f = lambda v: G.generalized_dot_product_attention(dev["q"], dev["k"], v, dev["qo"], dev["ko"], int(ln.max()),
                                                      int(ln.max()), qk_scale=scale, activation="gelu_approx").float()
    lhs = f((dev["v"].float() + v2.float()).to(torch.bfloat16))
    rhs = f(dev["v"]) + f(v2)
    assert G.kernel_status() == 0
    assert_close(lhs, rhs, "linearity in V", atol=ATOL, rtol=RTOL)


def test_host_errors_are_raised_before_any_launch(G):
    cpu, dev = jagged_inputs([10], [12], 1, 64, seed=1)
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 10, 12, activation="tanh")
    with pytest.raises(NotImplementedError):
        G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 10, 12, is_causal=True)
    with pytest.raises(TypeError):
        G.generalized_dot_product_attention(dev["q"].float(), dev["k"].float(), dev["v"].float(), dev["qo"], dev["ko"], 10, 12)
    q96 = torch.zeros(10, 1, 96, dtype=torch.bfloat16, device="cuda")
    k96 = torch.zeros(12, 1, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        G.generalized_dot_product_attention(q96, k96, k96, dev["qo"], dev["ko"], 10, 12)
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"][:1], 10, 12)


def test_bounded_wait_gives_up_and_reports_without_hanging(G):
    """A wait nothing satisfies runs out after its limit, writes a status code and returns; the
    context stays usable (the next operator call works)."""
    import ctypes as C

    from ads_model_kernel_library_b200.gdpa import _cabi

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _cabi.lib.gdpa_debug_wait_probe(C.c_void_p(status.data_ptr()), 20_000_000,  # 20 ms
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == (0x7700 | 1)
    assert _cabi.lib.gdpa_debug_wait_probe(None, 1000, None) == 1  # bad arguments are refused on the host
    cpu, dev = jagged_inputs([100], [100], 1, 64, seed=2, std=0.5)
    o = run_fwd(G, dev, [100], [100], "relu", 0.1)
    assert_close(o, oracle_forward(cpu, "relu", 0.1), "O after a timed-out probe")


def test_host_buffer_pipeline_matches_direct_call(G):
    """forward_backward_host (pinned host tensors, chunked, copies overlapped) == one direct call."""
    rng = np.random.default_rng(4)
    lq, lk = rng.integers(1, 400, 23), rng.integers(1, 500, 23)
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=13, std=0.5)
    o, dq, dk, dv = run_fwd_bwd(G, dev, lq, lk, "gelu_approx", 1.0 / 64)
    pinned = {n: cpu[n].pin_memory() for n in ("q", "k", "v", "do")}
    res = G.forward_backward_host(pinned["q"], pinned["k"], pinned["v"], pinned["do"], cpu["qo"], cpu["ko"],
                                  qk_scale=1.0 / 64, activation="gelu_approx", n_chunks=5)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    assert torch.equal(res["o"], o.cpu())
    assert torch.equal(res["dk"], dk.cpu()) and torch.equal(res["dv"], dv.cpu())
    assert_close(res["dq"], dq.float(), "dQ (host pipeline)", atol=1e-2, rtol=1e-2)


def test_flop_counter_mode_sees_the_operator(G):
    from torch.utils.flop_counter import FlopCounterMode

    lq, lk = [100, 37], [64, 200]
    cpu, dev = jagged_inputs(lq, lk, 2, 64, seed=3, std=0.5)
    q = dev["q"].clone().requires_grad_(True)
    with FlopCounterMode(display=False) as fc:
        o = G.generalized_dot_product_attention(q, dev["k"], dev["v"], dev["qo"], dev["ko"], 100, 200, activation="relu")
        o.backward(dev["do"])
    pairs = 100 * 64 + 37 * 200
    assert fc.get_total_flops() == 14 * 2 * 64 * pairs


def test_reduced_zipf_config5_shapes(G):
    """Heavily skewed lengths (32 * min(Zipf(1.2), 256), H=4, D=128, GELU-tanh): a reduced batch of the
    sharded configuration against the oracle, plus the two-shard split of it against the unsharded run."""
    from ads_model_kernel_library_b200.gdpa.sharding import shard_inputs

    rng = np.random.default_rng(5)
    ln = (32 * np.minimum(rng.zipf(1.2, 40), 256)).astype(np.int64)
    ln = np.minimum(ln, 2048)  # keep the CPU oracle in seconds
    cpu, dev = jagged_inputs(ln, ln, 4, 128, seed=55, std=0.5)
    scale = 1.0 / int(ln.max())
    o, dq, dk, dv = run_fwd_bwd(G, dev, ln, ln, "gelu_approx", scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "gelu_approx", scale)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)
    # token-balanced split in two: each shard alone reproduces its rows of the unsharded output bit for bit
    for rank in range(2):
        q_r, k_r, v_r, qo_r, ko_r, (s, e), (r0, r1) = shard_inputs(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], rank, 2)
        o_r = G.generalized_dot_product_attention(q_r.contiguous(), k_r.contiguous(), v_r.contiguous(), qo_r, ko_r,
                                                  int(ln[s:e].max()), int(ln[s:e].max()), qk_scale=scale,
                                                  activation="gelu_approx")
        assert torch.equal(o_r, o[r0:r1])


def test_many_heads_and_int32_offsets_backward(G):
    lq, lk = [150, 31, 260], [90, 300, 129]
    cpu, dev = jagged_inputs(lq, lk, 16, 64, seed=77, std=0.5, offset_dtype=torch.int32)
    o, dq, dk, dv = run_fwd_bwd(G, dev, lq, lk, "silu", 1.0 / 32)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "silu", 1.0 / 32)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)


@pytest.mark.parametrize("act", ["gelu_approx", "softmax"])
@pytest.mark.parametrize("hq,hkv", [(4, 1), (8, 2)])
def test_grouped_query_attention_forward_backward(G, act, hq, hkv):
    """H query heads share H_kv key/value heads (query head h reads K/V head h // group); dK and dV
    sum over the query heads of a group."""
    lq, lk = [130, 40, 257], [200, 129, 64]
    g = torch.Generator().manual_seed(91)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]))
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    q = (torch.randn(int(qo[-1]), hq, 128, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(int(ko[-1]), hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(int(ko[-1]), hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    do = (torch.randn(int(qo[-1]), hq, 128, generator=g) * 0.5).to(torch.bfloat16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = G.generalized_dot_product_attention(qd, kd, vd, qo.cuda(), ko.cuda(), max(lq), max(lk), qk_scale=0.1, activation=act)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    from oracle import gdpa_oracle as orc
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(q.float(), k.float(), v.float(), qo, ko, do.float(), act, 0.1)
    assert kd.grad.shape == k.shape and vd.grad.shape == v.shape
    for a, b, n in ((o, ro, "O"), (qd.grad, rdq, "dQ"), (kd.grad, rdk, "dK"), (vd.grad, rdv, "dV")):
        assert_close(a, b, f"{n}[gqa {hq}/{hkv} {act}]")


def test_shared_kv_sequences_via_ad_to_request_offset(G):
    """Many Q sequences ("ads") attend to the KV of one request: Q sequence i reads KV sequence
    ad_to_request_offset[i], as in the reference's inference path.  Forward only."""
    lq = [40, 130, 7, 260, 64]
    lk = [200, 90]                       # two requests
    ad2req = [0, 0, 1, 0, 1]
    g = torch.Generator().manual_seed(17)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]))
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    q = (torch.randn(int(qo[-1]), 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(int(ko[-1]), 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(int(ko[-1]), 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    o = G.generalized_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), qo.cuda(), ko.cuda(), max(lq), max(lk),
                                            ad_to_request_offset=torch.tensor(ad2req).cuda(), qk_scale=0.1,
                                            activation="gelu_approx")
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    from oracle import gdpa_oracle as orc
    # oracle: expand the shared KV into one KV sequence per ad
    k_exp = torch.cat([k[ko[r]:ko[r + 1]] for r in ad2req])
    v_exp = torch.cat([v[ko[r]:ko[r + 1]] for r in ad2req])
    ko_exp = torch.tensor(np.concatenate([[0], np.cumsum([lk[r] for r in ad2req])]))
    ref = orc.gdpa_forward(q.float(), k_exp.float(), v_exp.float(), qo, ko_exp, "gelu_approx", 0.1)
    assert_close(o, ref, "O[shared KV]")
    # the same with a band |q - kv| <= 20 of sequence-local positions
    ow = G.generalized_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), qo.cuda(), ko.cuda(), max(lq), max(lk),
                                             ad_to_request_offset=torch.tensor(ad2req).cuda(), qk_scale=0.1,
                                             activation="gelu_approx", window_size=20)
    torch.cuda.synchronize()
    refw = orc.gdpa_forward(q.float(), k_exp.float(), v_exp.float(), qo, ko_exp, "gelu_approx", 0.1, window_size=20)
    assert_close(ow, refw, "O[shared KV, banded]")
    qg = q.cuda().requires_grad_(True)
    og = G.generalized_dot_product_attention(qg, k.cuda(), v.cuda(), qo.cuda(), ko.cuda(), max(lq), max(lk),
                                             ad_to_request_offset=torch.tensor(ad2req).cuda(), activation="relu")
    with pytest.raises(NotImplementedError):
        og.backward(torch.ones_like(og))


def test_fused_qkv_and_fused_kv_layouts(G):
    """The reference's packed layouts: query = [T, H, 3D] with key = value = None (self-attention), and
    key = [T, H, 2D] with value = None.  The kernels read the slices in place; gradients flow back into
    the packed tensors."""
    ln = [70, 200, 129]
    off = torch.tensor(np.concatenate([[0], np.cumsum(ln)]))
    g = torch.Generator().manual_seed(23)
    qkv = (torch.randn(int(off[-1]), 2, 3 * 64, generator=g) * 0.5).to(torch.bfloat16)
    do = (torch.randn(int(off[-1]), 2, 64, generator=g) * 0.5).to(torch.bfloat16)
    from oracle import gdpa_oracle as orc

    q, k, v = qkv.float().split(64, dim=-1)
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(q, k, v, off, off, do.float(), "gelu_approx", 0.1)
    x = qkv.cuda().requires_grad_(True)
    o = G.generalized_dot_product_attention(x, None, None, off.cuda(), off.cuda(), max(ln), max(ln), qk_scale=0.1,
                                            activation="gelu_approx")
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    assert_close(o, ro, "O[fused QKV]")
    assert_close(x.grad, torch.cat([rdq, rdk, rdv], dim=-1), "d(QKV)")
    # fused KV with its own lengths
    lk = [90, 40, 260]
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    kv = (torch.randn(int(ko[-1]), 2, 2 * 64, generator=g) * 0.5).to(torch.bfloat16)
    qq = (torch.randn(int(off[-1]), 2, 64, generator=g) * 0.5).to(torch.bfloat16)
    k2, v2 = kv.float().split(64, dim=-1)
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(qq.float(), k2, v2, off, ko, do.float(), "silu", 0.1)
    xq, xkv = qq.cuda().requires_grad_(True), kv.cuda().requires_grad_(True)
    o = G.generalized_dot_product_attention(xq, xkv, None, off.cuda(), ko.cuda(), max(ln), max(lk), qk_scale=0.1,
                                            activation="silu")
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    assert_close(o, ro, "O[fused KV]")
    assert_close(xq.grad, rdq, "dQ[fused KV]")
    assert_close(xkv.grad, torch.cat([rdk, rdv], dim=-1), "d(KV)")


@pytest.mark.parametrize("act", ["gelu_approx", "softmax"])
@pytest.mark.parametrize("window", [0, 37, 200, 5000])
def test_banded_attention_window_size(G, act, window):
    """window_size = W keeps only pairs of sequence-local positions with |q - kv| <= W, forward and
    backward; a window wider than every sequence changes nothing."""
    lq, lk = [300, 70, 513, 129], [260, 200, 700, 131]
    cpu, dev = jagged_inputs(lq, lk, 2, 128, seed=61, std=0.5)
    from oracle import gdpa_oracle as orc

    q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=0.1, activation=act,
                                            window_size=window)
    o.backward(dev["do"])
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ro, rdq, rdk, rdv = orc.gdpa_forward_backward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"],
                                                  cpu["do"].float(), act, 0.1, window_size=window)
    for a, b, n in ((o, ro, "O"), (q.grad, rdq, "dQ"), (k.grad, rdk, "dK"), (v.grad, rdv, "dV")):
        assert_close(a, b, f"{n}[{act}, window {window}]")
    if window == 5000:
        o2 = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], max(lq), max(lk),
                                                 qk_scale=0.1, activation=act)
        assert torch.equal(o2, o)


@pytest.mark.parametrize("hq,hkv,ids", [
    (4, 4, [5, 5, 7]),          # relu, relu, silu, then the base activation for head 3
    (4, 2, [2, 2, 10, 10]),     # grouped-query, whole groups agree
    (4, 2, [2, 5, 5, 5, 9]),    # grouped-query, the first group is mixed; list longer than H is cut
])
def test_per_head_activations_ensemble(G, hq, hkv, ids):
    """ensemble_activation_list: head i < len(list) uses activation id list[i], the others the base."""
    lq, lk = [130, 40, 257], [200, 129, 64]
    g = torch.Generator().manual_seed(17)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]))
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    q = (torch.randn(int(qo[-1]), hq, 128, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(int(ko[-1]), hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(int(ko[-1]), hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    do = (torch.randn(int(qo[-1]), hq, 128, generator=g) * 0.5).to(torch.bfloat16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = G.generalized_dot_product_attention(qd, kd, vd, qo.cuda(), ko.cuda(), max(lq), max(lk), qk_scale=1.0 / 64,
                                            activation="gelu_approx", ensemble_activation_list=ids)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    from oracle import gdpa_oracle as orc
    from ads_model_kernel_library_b200.gdpa.math import int_to_activation
    names = [int_to_activation[ids[h]].value if h < len(ids) else "gelu_approx" for h in range(hq)]
    ro, rdq, rdk, rdv = orc.forward_backward_of(
        lambda a, b, c: orc.gdpa_forward_ensemble(a, b, c, qo, ko, names, 1.0 / 64), q.float(), k.float(), v.float(), do.float())
    assert o.shape == q.shape and o.is_contiguous()
    for a, b, n in ((o, ro, "O"), (qd.grad, rdq, "dQ"), (kd.grad, rdk, "dK"), (vd.grad, rdv, "dV")):
        assert_close(a, b, f"{n}[ensemble {ids}]")
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(qd, kd, vd, qo.cuda(), ko.cuda(), max(lq), max(lk),
                                            ensemble_activation_list=[42])


@pytest.mark.parametrize("act", ["gelu_approx", "softmax"])
def test_broadcast_q_one_query_sequence_for_the_batch(G, act):
    """broadcast_q: query holds one sequence; output [B * Lq, H, D], dQ summed over the batch."""
    LQ, lk, H = 150, [200, 129, 64, 1], 2
    g = torch.Generator().manual_seed(23)
    ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
    q = (torch.randn(LQ, H, 128, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(int(ko[-1]), H, 128, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(int(ko[-1]), H, 128, generator=g) * 0.5).to(torch.bfloat16)
    do = (torch.randn(len(lk) * LQ, H, 128, generator=g) * 0.5).to(torch.bfloat16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    qo = torch.tensor([0, LQ]).cuda()
    oo = (torch.arange(len(lk) + 1) * LQ).cuda()
    o = G.generalized_dot_product_attention(qd, kd, vd, qo, ko.cuda(), LQ, max(lk), qk_scale=0.1, activation=act,
                                            broadcast_q=True, output_offset=oo)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    from oracle import gdpa_oracle as orc
    ro, rdq, rdk, rdv = orc.forward_backward_of(
        lambda a, b, c: orc.gdpa_forward_broadcast_q(a, b, c, ko, act, 0.1), q.float(), k.float(), v.float(), do.float())
    assert o.shape == (len(lk) * LQ, H, 128) and qd.grad.shape == q.shape
    for a, b, n in ((o, ro, "O"), (qd.grad, rdq, "dQ"), (kd.grad, rdk, "dK"), (vd.grad, rdv, "dV")):
        assert_close(a, b, f"{n}[broadcast_q {act}]")
    o2 = G.generalized_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), qo, ko.cuda(), LQ, max(lk), qk_scale=0.1,
                                             activation=act, broadcast_q=True)
    assert torch.equal(o2, o)


@pytest.mark.parametrize("D,offset_dtype,act", [(128, torch.int64, "gelu_approx"), (64, torch.int32, "gelu_approx"),
                                                 (128, torch.int32, "softmax")])
def test_start_end_offsets_forward_backward(G, D, offset_dtype, act):
    """use_start_end_offsets: per-sequence [start, end] pairs; the K / V ranges of the sequences overlap (and one
    is shared outright), so dK / dV sum over every sequence that reads a row; one Q row belongs to no sequence."""
    H = 2
    q_pairs = [0, 300, 300, 429, 430, 431, 431, 700]     # row 429 is a gap; a one-row sequence
    k_pairs = [0, 260, 100, 500, 100, 500, 450, 777]     # overlaps; sequences 1 and 2 share one K / V range
    tq, tk = 700, 800                                    # K / V rows 777.. are read by nobody
    g = torch.Generator().manual_seed(91)
    q, do = (torch.randn(tq, H, D, generator=g) * 0.5).bfloat16(), (torch.randn(tq, H, D, generator=g) * 0.5).bfloat16()
    k, v = (torch.randn(tk, H, D, generator=g) * 0.5).bfloat16(), (torch.randn(tk, H, D, generator=g) * 0.5).bfloat16()
    qp = torch.tensor(q_pairs, dtype=offset_dtype, device="cuda")
    kp = torch.tensor(k_pairs, dtype=offset_dtype, device="cuda")
    mq = max(e - s for s, e in zip(q_pairs[0::2], q_pairs[1::2]))
    mk = max(e - s for s, e in zip(k_pairs[0::2], k_pairs[1::2]))
    scale = 0.5 if act == "softmax" else 1.0 / 64
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = G.generalized_dot_product_attention(qd, kd, vd, qp, kp, mq, mk, qk_scale=scale, activation=act,
                                            use_start_end_offsets=True, total_num_objects=tq)
    covered = torch.ones(tq, dtype=torch.bool)
    covered[429] = False
    o.backward(do.cuda() * covered.view(-1, 1, 1).cuda())
    torch.cuda.synchronize()
    assert G.kernel_status() == 0
    ro, rdq, rdk, rdv = orc.forward_backward_of(
        lambda a, b, c: orc.gdpa_forward_start_end(a, b, c, q_pairs, k_pairs, act, scale), q, k, v,
        do * covered.view(-1, 1, 1))
    assert_close(o[covered.cuda()], ro[covered], "O (start/end offsets)")
    assert_close(qd.grad, rdq, "dQ (start/end offsets)")
    assert_close(kd.grad, rdk, "dK (start/end offsets)")
    assert_close(vd.grad, rdv, "dV (start/end offsets)")
    assert float(kd.grad[777:].abs().max()) == 0.0 and float(qd.grad[429].abs().max()) == 0.0
    # the same batch written as prefix sums where that is possible (disjoint K / V): bit-identical forward
    qo = torch.tensor([0, 300, 700], dtype=offset_dtype, device="cuda")
    ko = torch.tensor([0, 260, 777], dtype=offset_dtype, device="cuda")
    a = G.generalized_dot_product_attention(qd.detach(), kd.detach(), vd.detach(), qo, ko, 400, 517, qk_scale=scale,
                                            activation="relu")
    b = G.generalized_dot_product_attention(qd.detach(), kd.detach(), vd.detach(),
                                            torch.tensor([0, 300, 300, 700], dtype=offset_dtype, device="cuda"),
                                            torch.tensor([0, 260, 260, 777], dtype=offset_dtype, device="cuda"), 400, 517,
                                            qk_scale=scale, activation="relu", use_start_end_offsets=True, total_num_objects=tq)
    assert torch.equal(a, b)


def test_start_end_offsets_argument_errors(G):
    q = torch.zeros(8, 2, 64, dtype=torch.bfloat16, device="cuda")
    pairs = torch.tensor([0, 8], device="cuda")
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(q, q, q, pairs, pairs, 8, 8, use_start_end_offsets=True)  # total_num_objects
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(q, q, q, pairs, pairs, 8, 8, use_start_end_offsets=True, total_num_objects=8,
                                            broadcast_q=True)
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(q, q, q, torch.tensor([0, 4, 8], device="cuda"),
                                            torch.tensor([0, 4, 8], device="cuda"), 8, 8, use_start_end_offsets=True,
                                            total_num_objects=8)  # an odd number of entries


def test_config5_longest_sequences_against_the_oracle(G):
    """The sharded Zipf configuration at its real lengths (H=4, D=128, GELU-tanh, scale 1/8192): one sequence at the
    8 192-token cap (64 KV tiles, 32 forward Q blocks: the heaviest bins of the schedule), one of 8 160 tokens (ragged
    last tile) and short ones in the same batch, forward and backward against the fp32 oracle."""
    ln = np.array([32, 8192, 96, 8160, 64, 544, 32, 1024], dtype=np.int64)
    cpu, dev = jagged_inputs(ln, ln, 4, 128, seed=56, std=0.5)
    scale = 1.0 / 8192
    o, dq, dk, dv = run_fwd_bwd(G, dev, ln, ln, "gelu_approx", scale)
    ro, rdq, rdk, rdv = oracle_forward_backward(cpu, "gelu_approx", scale)
    for a, b, n in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_close(a, b, n)


def test_offset_validation_is_opt_in_and_raises_before_any_launch(G):
    """With validation on, malformed offset arrays raise ValueError and nothing is launched; well-formed ones pass."""
    from ads_model_kernel_library_b200.gdpa import _cabi

    lq, lk = [100, 37], [64, 200]
    cpu, dev = jagged_inputs(lq, lk, 2, 64, seed=3, std=0.5)
    old = G.set_offset_validation(True)
    try:
        n0 = _cabi.lib.gdpa_launch_count()
        beyond = dev["qo"].clone(); beyond[-1] += 5            # last entry past the rows of the tensor
        down = dev["ko"].clone(); down[1] = down[2] + 1        # not monotone
        neg = dev["qo"].clone(); neg[0] = -1
        for qo, ko in ((beyond, dev["ko"]), (dev["qo"], down), (neg, dev["ko"])):
            with pytest.raises(ValueError):
                G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], qo, ko, 100, 200, activation="relu")
        with pytest.raises(ValueError):  # KV sequence index out of range
            G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 100, 200, activation="relu",
                                                ad_to_request_offset=torch.tensor([0, 2], device="cuda"))
        assert _cabi.lib.gdpa_launch_count() == n0
        o = G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 100, 200, qk_scale=0.1,
                                                activation="relu")
        assert_close(o, oracle_forward(cpu, "relu", 0.1), "O with validation on")
    finally:
        G.set_offset_validation(old)


def test_timed_out_wait_is_raised_by_the_next_operator_call(G):
    """The kernels' status word lives in pinned host memory: a wait that runs out (here the probe kernel's, with a
    20 ms limit, writing to the operator's own word) is reported by the next operator call on the device without
    anyone asking, and the call after that works."""
    import ctypes as C

    from ads_model_kernel_library_b200.gdpa import _cabi, ops

    cpu, dev = jagged_inputs([100], [100], 1, 64, seed=2, std=0.5)
    word = ops._status_word(dev["q"].device)
    assert word.is_pinned() and int(word[0]) == 0
    rc = _cabi.lib.gdpa_debug_wait_probe(C.c_void_p(word.data_ptr()), 20_000_000,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(word[0]) == (0x7700 | 1)  # written by the device straight into host memory
    with pytest.raises(RuntimeError, match="wait ran out"):
        G.generalized_dot_product_attention(dev["q"], dev["k"], dev["v"], dev["qo"], dev["ko"], 100, 100, activation="relu")
    o = run_fwd(G, dev, [100], [100], "relu", 0.1)  # the word was cleared by the raise
    assert_close(o, oracle_forward(cpu, "relu", 0.1), "O after a reported time-out")


def test_backward_schedule_can_be_reused_by_later_calls(G, monkeypatch):
    """The backward kernel draws its work items from a counter in the schedule header, which gdpa_bwd zeroes before
    every launch: a schedule built once serves any number of calls (one at a time).  Batches of fewer and of many more
    work items than the GPU has SMs."""
    from ads_model_kernel_library_b200.gdpa import ops

    built = {}
    real = ops._build_schedule

    def cached(mode, qo, ko, *rest, **kw):
        key = (mode, qo.data_ptr(), ko.data_ptr())
        if key not in built:
            built[key] = real(mode, qo, ko, *rest, **kw)
        return built[key]

    monkeypatch.setattr(ops, "_build_schedule", cached)
    for lens in ([300, 1, 129], list(np.random.default_rng(3).integers(1, 700, 96))):
        built.clear()
        cpu, dev = jagged_inputs(lens, lens, 4, 128, seed=11, std=0.5)
        lens = [int(x) for x in lens]
        ref = oracle_forward_backward(cpu, "gelu_approx", 1.0 / 128)
        grads = [run_fwd_bwd(G, dev, lens, lens, "gelu_approx", 1.0 / 128)[1:] for _ in range(3)]
        assert len(built) == 2  # one forward and one backward schedule, built once
        for g, e, name in zip(grads[-1], ref[1:], ("dq", "dk", "dv")):
            assert_close(g, e, name)
        # dK and dV are sums in a fixed order: identical from call to call; dQ is added up by reduce operations
        assert torch.equal(grads[0][1], grads[2][1]) and torch.equal(grads[0][2], grads[2][2])
        torch.testing.assert_close(grads[0][0].float(), grads[2][0].float(), atol=2e-2, rtol=2e-2)
