"""GPU tests of the MXFP8 wire format (e4m3 elements, e8m0 scale per 32 elements, 128-row padded scale atoms):
the quantiser and the de-quantiser are byte-exact against the CPU restatement, and the forward on MXFP8 inputs
matches the oracle evaluated on the de-quantised inputs at the bf16 bound (atol = rtol = 2e-2): the kernel
contracts exactly the de-quantised values and keeps P in bf16."""
import numpy as np
import pytest
import torch

from oracle import gdpa_oracle as orc
from tests._util import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import ads_model_kernel_library_b200.gdpa as g

    return g


def _jagged(lens, H, D, seed, dtype, spread=2.0):
    off = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(int(off[-1]), H, D, generator=g) * torch.exp(spread * torch.randn(int(off[-1]), H, 1, generator=g))
    return x.to(dtype), off


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype,offset_dtype,exact", [(torch.bfloat16, torch.int64, True), (torch.float32, torch.int32, False)])
def test_mxfp8_quantiser_matches_the_restatement_byte_for_byte(G, axis, D, dtype, offset_dtype, exact):
    lens = [130, 0, 5, 256, 1, 127, 33]
    x, off = _jagged(lens, 3, D, seed=17 + axis, dtype=dtype)
    x[7, 1] = 0  # an all-zero block: code 0, elements 0
    x8, sf, cu = G.quantize_varlen_mxfp8_sf_only(x.cuda(), off.to(offset_dtype).cuda(), scale_axis=axis, exact_layout=exact)
    torch.cuda.synchronize()
    blocks = sum((n + 127) // 128 for n in lens)
    sf_blocks = blocks if exact else int(off[-1]) // 128 + len(lens)
    r8, rsf, rcu = orc.quantize_mxfp8(x.float(), off, axis, sf_blocks=sf_blocks)
    assert cu.dtype == torch.int32 and cu.cpu().tolist() == rcu.tolist()
    assert sf.dtype == torch.float8_e8m0fnu and sf.numel() == rsf.numel()
    assert torch.equal(x8.cpu().view(torch.uint8), r8.view(torch.uint8))
    assert torch.equal(sf.cpu().view(torch.uint8).reshape(-1), rsf)
    # and back: the values the kernels contract, exact in bf16 and in fp32
    want = orc.dequantize_mxfp8(r8, rsf, off, axis, sf_blocks=sf_blocks)
    for out_dtype in (torch.bfloat16, torch.float32):
        y = G.dequantize_mxfp8(x8, sf, off.to(offset_dtype).cuda(), scale_axis=axis, dtype=out_dtype)
        torch.cuda.synchronize()
        if out_dtype == torch.bfloat16:  # bf16 holds every e4m3 value times a power of two in its normal range
            ok = want.abs() >= 2.0 ** -126
            assert torch.equal(y.float().cpu()[ok], want[ok])
        else:
            assert torch.equal(y.cpu(), want)


def test_mxfp8_empty_batch(G):
    x = torch.zeros(0, 2, 128, dtype=torch.bfloat16, device="cuda")
    off = torch.zeros(1, dtype=torch.int64, device="cuda")
    x8, sf, cu = G.quantize_varlen_mxfp8_sf_only(x, off)
    assert x8.shape == (0, 2, 128) and cu.cpu().tolist() == [0]
    assert G.dequantize_mxfp8(x8, sf, off).shape == (0, 2, 128)


def test_mxfp8_argument_errors(G):
    x = torch.zeros(4, 2, 48, dtype=torch.bfloat16, device="cuda")
    off = torch.tensor([0, 4], device="cuda")
    with pytest.raises(ValueError):
        G.quantize_varlen_mxfp8_sf_only(x, off)  # head_dim not a multiple of 32
    with pytest.raises(ValueError):
        G.quantize_varlen_mxfp8_sf_only(torch.zeros(4, 2, 64, device="cuda", dtype=torch.float16), off)
    with pytest.raises(ValueError):
        G.quantize_varlen_mxfp8_sf_only(torch.zeros(4, 2, 64, device="cuda"), off, scale_axis=2)


@pytest.mark.parametrize("activation,scale", [("softmax", 0.0883883), ("gelu_approx", 1.0 / 300), ("relu", None)])
def test_mxfp8_forward_matches_oracle_on_dequantised_inputs(G, activation, scale):
    lq, lk = [1, 70, 300, 129, 256], [5, 200, 131, 260, 77]
    H, D = 2, 128
    q, qo = _jagged(lq, H, D, 41, torch.bfloat16, spread=0.5)
    k, ko = _jagged(lk, H, D, 42, torch.bfloat16, spread=0.5)
    v, _ = _jagged(lk, H, D, 43, torch.bfloat16, spread=0.5)
    if activation == "relu":  # keep |O| of the unscaled relu near 1
        q, k = q * 0.05, k * 0.05
    qo_d, ko_d = qo.cuda(), ko.cuda()
    q8, sfq, cuq = G.quantize_varlen_mxfp8_sf_only(q.cuda(), qo_d, 0)
    k8, sfk, cuk = G.quantize_varlen_mxfp8_sf_only(k.cuda(), ko_d, 0)
    v8, sfv, _ = G.quantize_varlen_mxfp8_sf_only(v.cuda(), ko_d, 1)
    o = G.generalized_dot_product_attention_mxfp8(q8, k8, v8, sfq, sfk, sfv, qo_d, ko_d, max(lq), max(lk), qk_scale=scale,
                                                  activation=activation, cu_seqlens_sf_q=cuq, cu_seqlens_sf_k=cuk)
    torch.cuda.synchronize()
    assert G.kernel_status() == 0 and o.dtype == torch.bfloat16
    deq = [orc.dequantize_mxfp8(*orc.quantize_mxfp8(t.float(), off, ax)[:2], off, ax)
           for t, off, ax in ((q, qo, 0), (k, ko, 0), (v, ko, 1))]
    ref = orc.gdpa_forward(deq[0], deq[1], deq[2], qo, ko, activation, scale)
    assert_close(o, ref, f"O[mxfp8 {activation}]")
