"""The operator inside a CUDA graph and inside torch.compile: what the reference's callers rely on (the entry point
is `@torch.fx.wrap`ped and registered with fake kernels, gdpa/triton/triton_generalized_dot_product_attention.py:4229,
:3099-3335) and what the boundary promises (no host synchronisation, nothing allocated by the library)."""
import pytest
import torch

from tests._util import jagged_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


def _fwd_bwd(G, q, k, v, do, qo, ko, mq, mk, act, scale):
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    o = G.generalized_dot_product_attention(q, k, v, qo, ko, mq, mk, qk_scale=scale, activation=act)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    return o, dq, dk, dv


@pytest.mark.parametrize("act", ["gelu_approx", "softmax"])
def test_forward_and_backward_replay_from_a_cuda_graph(G, act):
    lq, lk = [130, 1, 257, 64], [200, 77, 129, 300]
    _, dev = jagged_inputs(lq, lk, 2, 128, seed=71, std=0.5)
    _, other = jagged_inputs(lq, lk, 2, 128, seed=72, std=0.5)
    args = (dev["qo"], dev["ko"], max(lq), max(lk), act, 1.0 / 64)
    static = {n: dev[n].clone() for n in ("q", "k", "v", "do")}
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (per-device attribute cache, allocator pools)
        _fwd_bwd(G, static["q"], static["k"], static["v"], static["do"], *args)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = _fwd_bwd(G, static["q"], static["k"], static["v"], static["do"], *args)
    for src in (dev, other):  # replay on two different inputs written into the captured buffers
        for n in static:
            static[n].copy_(src[n])
        graph.replay()
        torch.cuda.synchronize()
        assert G.kernel_status() == 0
        want = _fwd_bwd(G, src["q"], src["k"], src["v"], src["do"], *args)
        torch.cuda.synchronize()
        for got, ref, name in zip(outs, want, ("O", "dQ", "dK", "dV")):
            if name == "dQ":  # fp32 reduce-adds arrive in a different order from run to run
                torch.testing.assert_close(got.float(), ref.float(), atol=1e-2, rtol=1e-2)
            else:
                assert torch.equal(got, ref), name


def test_operator_traces_under_torch_compile(G):
    """aot_eager: dynamo + AOT autograd trace through the fake kernels and the registered backward, then run the real
    kernels; the compiled function gives the eager function's results bit for bit (dQ up to its reduction order)."""
    lq, lk = [100, 37, 300], [64, 200, 131]
    _, dev = jagged_inputs(lq, lk, 2, 64, seed=9, std=0.5)

    def fn(q, k, v):
        o = G.generalized_dot_product_attention(q, k, v, dev["qo"], dev["ko"], max(lq), max(lk), qk_scale=1.0 / 64,
                                                activation="silu")
        return o * 2.0

    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    res = []
    for f in (fn, compiled):
        q, k, v = (dev[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
        y = f(q, k, v)
        y.backward(dev["do"])
        torch.cuda.synchronize()
        res.append((y.detach(), q.grad, k.grad, v.grad))
    assert G.kernel_status() == 0
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][2], res[1][2]) and torch.equal(res[0][3], res[1][3])
    torch.testing.assert_close(res[0][1].float(), res[1][1].float(), atol=1e-2, rtol=1e-2)
