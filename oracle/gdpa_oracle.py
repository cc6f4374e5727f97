"""CPU oracle for GDPA (Generalized Dot Product Attention). TEST INFRASTRUCTURE ONLY.

This file restates, in eager PyTorch fp32 on the CPU, the algorithm the reference library
defines for jagged GDPA.  It exists so that the CUDA kernels can be checked against it; it is
never imported by the shipped package (only by tests, the smoke check and the CPU-baseline leg
of the benchmark).

Parity pin: the reference stores no golden tensors for this path.  The restatement is pinned
against outputs of the reference's own Python code run on the CPU (committed under
``tests/golden/`` together with the script that produced them):

* ``cpu_generalized_dot_product_attention`` (softmax, no scale, separate Q / KV offsets),
  gdpa/triton/triton_generalized_dot_product_attention.py:3898-3979;
* the eager helper ``_gdpa_reference`` (act(q kT) v per sequence, fp32),
  gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:35-47, with the activation table
  ``get_pytorch_activation``, gdpa/triton/math.py:58-74.

* the reference's Triton forward and backward kernels themselves
  (gdpa/triton/triton_generalized_dot_product_attention.py:3099-3335, :3461-3788) executed on the CPU
  by Triton's interpreter, with ``qk_scale = 0.25``, different Q and KV lengths and a grouped-query
  case: O, dQ, dK, dV for raw, gelu_approx, leaky_relu, relu, silu, hardswish, relu_square (the other
  activations are written with inline PTX, which the interpreter cannot run).

The last item pins where ``qk_scale`` is applied (``p = act(qk); p *= qk_scale``, :279-307) and every
gradient (``dS = qk_scale * act'(S) * dP``, :1626-1634); gradients here come from autograd over the
forward below, which is the same chain rule.  Not pinned by reference outputs: the softmax backward
(the reference has none) and the FP8 block-scaled variant (no CPU or interpreter path in the
reference); both are checked against this fp32 restatement only.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

# Activation names and integer ids of the reference, in enumeration order
# (gdpa/triton/math.py:43-55 and :77-78).  "softmax" is not in the reference enum; it is the
# name this library gives to the behaviour of the reference's CPU kernel.
ACTIVATION_IDS: Dict[str, int] = {
    "raw": 0,
    "gelu": 1,
    "gelu_approx": 2,
    "fast_gelu": 3,
    "leaky_relu": 4,
    "relu": 5,
    "fast_gelu_bf16": 6,
    "silu": 7,
    "fast_silu": 8,
    "hardswish": 9,
    "relu_square": 10,
    "fast_gelu_taylor_approx": 11,
}


def pytorch_activation(name: str) -> Callable[[torch.Tensor], torch.Tensor]:
    """Eager activation for a reference activation name (gdpa/triton/math.py:58-74)."""
    if name not in ACTIVATION_IDS:
        # same error class and wording as activation_string_to_int, gdpa/triton/math.py:81-85
        raise ValueError(f"Unsupported activation function: {name}")
    if name == "raw":
        return lambda x: x
    if name == "gelu":
        return lambda x: F.gelu(x)
    if name in ("gelu_approx", "fast_gelu", "fast_gelu_bf16", "fast_gelu_taylor_approx"):
        return lambda x: F.gelu(x, approximate="tanh")
    if name == "leaky_relu":
        return lambda x: F.leaky_relu(x, 0.01)
    if name == "relu":
        return torch.relu
    if name in ("silu", "fast_silu"):
        return F.silu
    if name == "hardswish":
        return F.hardswish
    if name == "relu_square":
        return lambda x: torch.relu(x) * torch.relu(x)
    raise AssertionError(name)


def gdpa_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    activation: str = "raw",
    qk_scale: Optional[float] = None,
    p_dtype: Optional[torch.dtype] = None,
    window_size: Optional[int] = None,
) -> torch.Tensor:
    """O[b] = (act(Q_b K_b^T) * qk_scale) V_b per sequence and head, in fp32.

    Loop, slicing and transposes follow cpu_generalized_dot_product_attention
    (gdpa/triton/triton_generalized_dot_product_attention.py:3950-3979); the activation and the
    post-activation scale follow the device kernel (:279-307).  ``activation="softmax"``
    computes softmax(qk_scale * S) V, which for ``qk_scale=None`` is exactly the reference CPU
    kernel (:3973-3975).

    ``p_dtype`` optionally rounds P to that dtype before the second contraction, as the device
    kernels do (:307); the default keeps fp32 throughout.
    """
    scale = 1.0 if qk_scale is None else float(qk_scale)  # :3148-3149
    q = query.to(torch.float32)
    k = key.to(torch.float32)
    v = value.to(torch.float32)
    out = torch.zeros_like(q)
    bs = query_offset.numel() - 1
    act = None if activation == "softmax" else pytorch_activation(activation)
    for i in range(bs):
        qs, qe = int(query_offset[i]), int(query_offset[i + 1])
        ks, ke = int(key_offset[i]), int(key_offset[i + 1])
        if qe <= qs:
            continue
        q_i = q[qs:qe].transpose(0, 1)  # [H, Lq, D]
        k_i = k[ks:ke].transpose(0, 1)
        v_i = v[ks:ke].transpose(0, 1)
        if k_i.shape[0] != q_i.shape[0]:
            # grouped-query attention: query head h reads K / V head h // group
            # (off_h_kv = off_h // G, gdpa/triton/triton_generalized_dot_product_attention.py:954)
            group = q_i.shape[0] // k_i.shape[0]
            k_i = k_i.repeat_interleave(group, dim=0)
            v_i = v_i.repeat_interleave(group, dim=0)
        s = torch.matmul(q_i, k_i.transpose(-2, -1))
        band = None
        if window_size is not None:
            # |q - kv| <= window_size on sequence-local positions; scores outside are zeroed before the
            # activation (gdpa/triton/triton_generalized_dot_product_attention.py:274-278)
            pos_q = torch.arange(qe - qs).view(-1, 1)
            pos_k = torch.arange(ke - ks).view(1, -1)
            band = (pos_q - pos_k).abs() <= int(window_size)
        if act is None:
            if ke > ks:
                sc = s * scale
                if band is not None:
                    sc = sc.masked_fill(~band, float("-inf"))
                p = torch.nan_to_num(F.softmax(sc, dim=-1), nan=0.0)  # a row without keys in its band gives zeros
            else:
                p = s
        else:
            if band is not None:
                s = torch.where(band, s, torch.zeros_like(s))
            p = act(s) * scale
        if p_dtype is not None:
            p = p.to(p_dtype).to(torch.float32)
        o_i = torch.matmul(p, v_i)
        out[qs:qe] = o_i.transpose(0, 1)
    return out


def gdpa_forward_backward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    grad_out: torch.Tensor,
    activation: str = "raw",
    qk_scale: Optional[float] = None,
    window_size: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(O, dQ, dK, dV) in fp32 by autograd over :func:`gdpa_forward`.

    Equivalent to the hand formulas of the reference backward: dP = dO V^T,
    dS = qk_scale act'(S) dP, dV = (qk_scale act(S))^T dO, dK = dS^T Q, dQ = dS K
    (gdpa/triton/triton_generalized_dot_product_attention.py:1602-1634, :1761-1805).
    """
    q = query.detach().to(torch.float32).clone().requires_grad_(True)
    k = key.detach().to(torch.float32).clone().requires_grad_(True)
    v = value.detach().to(torch.float32).clone().requires_grad_(True)
    o = gdpa_forward(q, k, v, query_offset, key_offset, activation, qk_scale, window_size=window_size)
    o.backward(grad_out.to(torch.float32))
    zero = torch.zeros_like
    return (
        o.detach(),
        q.grad if q.grad is not None else zero(q),
        k.grad if k.grad is not None else zero(k),
        v.grad if v.grad is not None else zero(v),
    )


def gdpa_forward_ensemble(query, key, value, query_offset, key_offset, activations, qk_scale=None, window_size=None):
    """Per-head activations: head h uses ``activations[h]`` (the reference's ensemble_activation_list,
    gdpa/triton/triton_generalized_dot_product_attention.py:958-961, backward :2686-2688).  One
    :func:`gdpa_forward` per query head, concatenated; differentiable."""
    H, Hkv = query.shape[1], key.shape[1]
    G = H // Hkv
    outs = [
        gdpa_forward(query[:, h:h + 1], key[:, h // G:h // G + 1], value[:, h // G:h // G + 1], query_offset, key_offset,
                     activations[h], qk_scale, window_size=window_size)
        for h in range(H)
    ]
    return torch.cat(outs, dim=1)


def gdpa_forward_broadcast_q(query, key, value, key_offset, activation="raw", qk_scale=None):
    """``broadcast_q``: the single Q sequence ``query`` ([Lq, H, D]) attends with every KV sequence of the batch;
    output ``[B * Lq, H, D]`` with the rows of batch element z at z * Lq (off_q_z = 0 at
    gdpa/triton/triton_generalized_dot_product_attention.py:949-952; output shape :3028).  Differentiable:
    dQ sums over the batch, as the reference's atomic adds do (:2582-2583)."""
    lq = query.shape[0]
    qo = torch.tensor([0, lq])
    outs = []
    for z in range(key_offset.numel() - 1):
        ks, ke = int(key_offset[z]), int(key_offset[z + 1])
        outs.append(gdpa_forward(query, key[ks:ke], value[ks:ke], qo, torch.tensor([0, ke - ks]), activation, qk_scale))
    return torch.cat(outs, dim=0)


def gdpa_forward_start_end(query, key, value, query_pairs, key_pairs, activation="raw", qk_scale=None):
    """The reference's ``use_start_end_offsets`` (gdpa/triton/triton_generalized_dot_product_attention.py:943-946,
    :599-618, :4270-4274): offsets are ``[start_0, end_0, start_1, end_1, ...]``, sequence ``b`` reads Q rows
    ``[q_pairs[2b], q_pairs[2b+1])`` and K / V rows ``[k_pairs[2b], k_pairs[2b+1])`` (which may overlap between
    sequences) and writes the output rows of its Q range; rows no sequence owns stay zero.  Built from torch ops so
    that autograd gives the gradients, dK / dV summed over the sequences that read a row."""
    act = None if activation == "softmax" else pytorch_activation(activation)
    scale = 1.0 if qk_scale is None else float(qk_scale)
    qp = [int(x) for x in query_pairs]
    kp = [int(x) for x in key_pairs]
    out = torch.zeros_like(query)
    pieces = []
    for b in range(len(qp) // 2):
        qs, qe, ks, ke = qp[2 * b], qp[2 * b + 1], kp[2 * b], kp[2 * b + 1]
        if qe <= qs:
            continue
        qb = query[qs:qe].transpose(0, 1)
        kb = key[ks:ke].transpose(0, 1)
        vb = value[ks:ke].transpose(0, 1)
        sc = torch.matmul(qb, kb.transpose(-1, -2))
        p = F.softmax(sc * scale, dim=-1) if act is None else act(sc) * scale
        pieces.append((qs, qe, torch.matmul(p, vb).transpose(0, 1)))
    for qs, qe, ob in pieces:
        out = torch.cat([out[:qs], ob, out[qe:]], dim=0)
    return out


def forward_backward_of(fn, query, key, value, grad_out):
    """(O, dQ, dK, dV) in fp32 by autograd over ``fn(q, k, v)``, for the composed variants above."""
    q = query.detach().to(torch.float32).clone().requires_grad_(True)
    k = key.detach().to(torch.float32).clone().requires_grad_(True)
    v = value.detach().to(torch.float32).clone().requires_grad_(True)
    o = fn(q, k, v)
    o.backward(grad_out.to(torch.float32))
    zero = torch.zeros_like
    return (o.detach(), q.grad if q.grad is not None else zero(q), k.grad if k.grad is not None else zero(k),
            v.grad if v.grad is not None else zero(v))


def gdpa_with_norms(query, key, value, query_offset, key_offset, activation="fast_gelu", qk_scale=None,
                    fused_layernorm=False, layernorm_weight=None, layernorm_bias=None, fused_q_residual_add=False,
                    fused_rms_norm=False, rms_norm_weight=None, residual=None, round_dtype=None, eps=1e-5):
    """The reference's GDPA-plus-norm pipeline, forward, in fp32:
    ``q' = LayerNorm(query)`` over heads * head_dim (rounded to ``round_dtype`` like the reference, which keeps it
    in the input dtype), ``x = GDPA(q', K, V) [+ q']``, ``y = x * rsqrt(mean(x^2) + eps) [* w]``, ``[+ residual]``.
    Follows the eager formulation of gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:67-74 and :110-127 and the
    order of the kernel epilogue (gdpa_megakernel/src/tlx_gdpa_megakernel.py:1076-1142: Q residual before the
    norm, generic residual after it; eps 1e-5 at :402 and :481)."""
    T, H, D = query.shape
    q = query.to(torch.float32)
    if fused_layernorm:
        w = None if layernorm_weight is None else layernorm_weight.to(torch.float32).reshape(H * D)
        b = None if layernorm_bias is None else layernorm_bias.to(torch.float32).reshape(H * D)
        q = torch.nn.functional.layer_norm(q.reshape(T, H * D), (H * D,), w, b, eps).reshape(T, H, D)
        if round_dtype is not None:
            q = q.to(round_dtype).to(torch.float32)
    x = gdpa_forward(q, key, value, query_offset, key_offset, activation, qk_scale)
    if fused_q_residual_add:
        x = x + q
    if fused_rms_norm:
        x2 = x.reshape(T, H * D)
        x2 = x2 * torch.rsqrt(x2.pow(2).mean(dim=1, keepdim=True) + eps)
        if rms_norm_weight is not None:
            x2 = x2 * rms_norm_weight.to(torch.float32).reshape(1, H * D)
        x = x2.reshape(T, H, D)
    if residual is not None:
        x = x + residual.to(torch.float32)
    return x


def quantize_fp8_blockwise(x: torch.Tensor, offsets: torch.Tensor):
    """CPU restatement of this library's FP8 input format (no counterpart in the reference, whose quantisation
    helper is missing from its tree): one fp32 scale per (sequence-local 128-token block, head),
    ``scale = max(amax / 448, 1e-12)``, ``x8 = e4m3(clamp(x / scale, -448, 448))``.  Returns
    ``(x8, scales[num_blocks, H], block_offsets[B + 1])``."""
    off = offsets.to(torch.int64).cpu()
    lens = (off[1:] - off[:-1]).clamp_min(0)
    nblk = (lens + 127) // 128
    blk_off = torch.zeros(off.numel(), dtype=torch.int64)
    blk_off[1:] = torch.cumsum(nblk, 0)
    total, H, D = x.shape
    xf = x.detach().cpu().to(torch.float32)
    scales = torch.zeros(int(blk_off[-1]), H, dtype=torch.float32)
    x8 = torch.empty(total, H, D, dtype=torch.float8_e4m3fn)
    for b in range(lens.numel()):
        s, e = int(off[b]), int(off[b + 1])
        for j, r0 in enumerate(range(s, e, 128)):
            blk = xf[r0:min(r0 + 128, e)]
            sc = (blk.abs().amax(dim=(0, 2)) / 448.0).clamp_min(1e-12)
            scales[int(blk_off[b]) + j] = sc
            x8[r0:min(r0 + 128, e)] = (blk / sc.view(1, H, 1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return x8, scales, blk_off.to(offsets.dtype)


def mx_e8m0_codes(amax: torch.Tensor) -> torch.Tensor:
    """e8m0 code (uint8 held in int64) of blocks with absolute maxima ``amax`` (fp32) by the reference's round-up rule
    for its P tile (gdpa/src/activation_utils.py:444-517): ``t = amax * (1 / 448)`` in fp32, the exponent field of
    ``t``, plus one when the mantissa of ``t`` is not zero; 255 (the NaN code) is clamped to 254."""
    t = (amax.to(torch.float32) * torch.tensor(1.0 / 448.0, dtype=torch.float32)).contiguous()
    bits = t.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    e = (bits >> 23) & 0xFF
    e = e + ((bits & 0x7FFFFF) != 0).to(torch.int64)
    return e.clamp_max(254)


def mx_scale_atom_byte(row: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """Byte inside a 512-byte scale atom (128 rows x 4 scales) of row ``row`` (0..127) and 32-element block ``k``
    (0..3): the layout the reference builds with ``tile_atom_to_shape_SF`` (gdpa/src/flash_fwd_sm100.py:746-833)."""
    return 16 * (row % 32) + 4 * (row // 32) + k


def _mx_block_offsets(offsets: torch.Tensor) -> torch.Tensor:
    off = offsets.to(torch.int64).cpu()
    nblk = ((off[1:] - off[:-1]).clamp_min(0) + 127) // 128
    blk_off = torch.zeros(off.numel(), dtype=torch.int64)
    blk_off[1:] = torch.cumsum(nblk, 0)
    return blk_off


def quantize_mxfp8(x: torch.Tensor, offsets: torch.Tensor, scale_axis: int = 0, sf_blocks: Optional[int] = None):
    """CPU restatement of the MXFP8 wire format of the reference's block-scaled variant (element tensor unpadded,
    scale tensor padded per sequence to 128 rows: gdpa/src/interface.py:714-750): e4m3 elements, one e8m0 scale per
    32 elements along the head dim (``scale_axis=0``: Q, K) or along the tokens (``scale_axis=1``: V).
    Returns ``(x8, sf, cu_seqlens_sf)``: ``sf`` is a flat uint8 tensor of 512-byte atoms ordered
    [head][token block][head-dim atom] (axis 0) or [head][head-dim atom][token block] (axis 1), ``sf_blocks`` token
    blocks per head (default: exactly the blocks of the batch), zero where no element exists."""
    off = offsets.to(torch.int64).cpu()
    blk_off = _mx_block_offsets(offsets)
    nblocks = int(blk_off[-1])
    sf_blocks = nblocks if sf_blocks is None else int(sf_blocks)
    total, H, D = x.shape
    d_atoms = (D + 127) // 128
    xf = x.detach().cpu().to(torch.float32)
    x8 = torch.zeros(total, H, D, dtype=torch.float8_e4m3fn)
    sf = torch.zeros(H * d_atoms * sf_blocks * 512, dtype=torch.uint8)
    hs = torch.arange(H)
    for b in range(off.numel() - 1):
        s, e = int(off[b]), int(off[b + 1])
        for j, r0 in enumerate(range(s, e, 128)):
            g = int(blk_off[b]) + j
            blk = xf[r0:min(r0 + 128, e)]  # [n, H, D]
            n = blk.shape[0]
            if scale_axis == 0:
                v = blk.reshape(n, H, D // 32, 32)
                codes = mx_e8m0_codes(v.abs().amax(dim=-1))  # [n, H, D/32]
                inv = torch.pow(2.0, (127 - codes).to(torch.float64)).to(torch.float32)
                q = (v * inv.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
                x8[r0:r0 + n] = q.reshape(n, H, D)
                rows = torch.arange(n).view(n, 1, 1)
                kb = torch.arange(D // 32).view(1, 1, -1)
                atom = (hs.view(1, H, 1) * sf_blocks + g) * d_atoms + kb // 4
                sf[(atom * 512 + mx_scale_atom_byte(rows, kb % 4)).reshape(-1)] = codes.reshape(-1).to(torch.uint8)
            else:
                pad = torch.zeros(128, H, D)
                pad[:n] = blk
                v = pad.reshape(4, 32, H, D)
                codes = mx_e8m0_codes(v.abs().amax(dim=1))  # [4, H, D]
                inv = torch.pow(2.0, (127 - codes).to(torch.float64)).to(torch.float32)
                q = (v * inv.unsqueeze(1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(128, H, D)
                x8[r0:r0 + n] = q[:n]
                live = (torch.arange(4) * 32 < n).view(4, 1, 1).expand(4, H, D)  # 32-token blocks that hold a token
                kb = torch.arange(4).view(4, 1, 1)
                d = torch.arange(D).view(1, 1, D)
                atom = (hs.view(1, H, 1) * d_atoms + d // 128) * sf_blocks + g
                idx = (atom * 512 + mx_scale_atom_byte(d % 128, kb)).expand(4, H, D)
                sf[idx[live]] = codes[live].to(torch.uint8)
    return x8, sf, (blk_off * 128).to(torch.int32)


def dequantize_mxfp8(x8: torch.Tensor, sf: torch.Tensor, offsets: torch.Tensor, scale_axis: int = 0,
                     sf_blocks: Optional[int] = None) -> torch.Tensor:
    """fp32 values of an MXFP8 tensor in the layout of :func:`quantize_mxfp8`: element * 2^(code - 127)."""
    off = offsets.to(torch.int64).cpu()
    blk_off = _mx_block_offsets(offsets)
    total, H, D = x8.shape
    d_atoms = (D + 127) // 128
    sf_blocks = int(blk_off[-1]) if sf_blocks is None else int(sf_blocks)
    sfl = sf.cpu().to(torch.int64)
    xf = x8.cpu().to(torch.float32)
    out = torch.zeros(total, H, D, dtype=torch.float32)
    hs = torch.arange(H).view(1, H, 1)
    d = torch.arange(D).view(1, 1, D)
    for b in range(off.numel() - 1):
        s, e = int(off[b]), int(off[b + 1])
        if e <= s:
            continue
        t = torch.arange(e - s).view(-1, 1, 1)
        g = int(blk_off[b]) + t // 128
        if scale_axis == 0:
            atom = (hs * sf_blocks + g) * d_atoms + d // 128
            byte = mx_scale_atom_byte(t % 128, (d % 128) // 32)
        else:
            atom = (hs * d_atoms + d // 128) * sf_blocks + g
            byte = mx_scale_atom_byte(d % 128, (t % 128) // 32)
        codes = sfl[(atom * 512 + byte).reshape(-1)].reshape(e - s, H, D)
        out[s:e] = (xf[s:e].to(torch.float64) * torch.pow(2.0, (codes - 127).to(torch.float64))).to(torch.float32)
    return out


def gdpa_backward_formulas(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    grad_out: torch.Tensor,
    activation: str,
    qk_scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dQ, dK, dV) from the closed-form derivative tables of the reference
    (gdpa/triton/math.py:196-206 tanh-GELU, :359-367 SiLU, relu / raw / relu_square / leaky_relu
    / hardswish / erf-GELU likewise), used to cross-check the autograd route on the CPU."""
    scale = 1.0 if qk_scale is None else float(qk_scale)
    q = query.to(torch.float32)
    k = key.to(torch.float32)
    v = value.to(torch.float32)
    do = grad_out.to(torch.float32)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for i in range(query_offset.numel() - 1):
        qs, qe = int(query_offset[i]), int(query_offset[i + 1])
        ks, ke = int(key_offset[i]), int(key_offset[i + 1])
        if qe <= qs or ke <= ks:
            continue
        q_i = q[qs:qe].transpose(0, 1)
        k_i = k[ks:ke].transpose(0, 1)
        v_i = v[ks:ke].transpose(0, 1)
        do_i = do[qs:qe].transpose(0, 1)
        s = q_i @ k_i.transpose(-2, -1)
        p, dact = activation_and_grad(s, activation)
        dp = do_i @ v_i.transpose(-2, -1)
        ds = dact * dp * scale
        dv[ks:ke] = ((p * scale).transpose(-2, -1) @ do_i).transpose(0, 1)
        dk[ks:ke] = (ds.transpose(-2, -1) @ q_i).transpose(0, 1)
        dq[qs:qe] = (ds @ k_i).transpose(0, 1)
    return dq, dk, dv


def activation_and_grad(x: torch.Tensor, name: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """act(x) and act'(x) from the reference's closed forms (gdpa/triton/math.py:99-413)."""
    if name == "raw":
        return x, torch.ones_like(x)
    if name == "relu":
        return torch.relu(x), (x > 0).to(x.dtype)
    if name == "leaky_relu":
        return F.leaky_relu(x, 0.01), torch.where(x > 0, 1.0, 0.01).to(x.dtype)
    if name == "relu_square":
        r = torch.relu(x)
        return r * r, 2.0 * r
    if name in ("gelu_approx", "fast_gelu", "fast_gelu_bf16", "fast_gelu_taylor_approx"):
        c0, c1 = 0.7978845608028654, 0.044715
        t = torch.tanh(c0 * x * (1.0 + c1 * x * x))
        return 0.5 * x * (1.0 + t), 0.5 * x * (1.0 - t * t) * (c0 + 3.0 * c0 * c1 * x * x) + 0.5 * (1.0 + t)
    if name == "gelu":
        cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
        pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
        return x * cdf, cdf + x * pdf
    if name in ("silu", "fast_silu"):
        sg = torch.sigmoid(x)
        return x * sg, sg * (1.0 + x * (1.0 - sg))
    if name == "hardswish":
        y = F.hardswish(x)
        g = torch.where(x < -3.0, 0.0, torch.where(x > 3.0, 1.0, (2.0 * x + 3.0) / 6.0))
        return y, g.to(x.dtype)
    raise ValueError(f"Unsupported activation function: {name}")


def useful_flops(q_lens: Sequence[int], kv_lens: Sequence[int], heads: int, head_dim: int, mode: str = "fwd") -> int:
    """Useful FLOPs over valid jagged pairs only: 4 H D sum(Lq Lkv) forward, x2.5 backward,
    x3.5 forward+backward (gdpa/scripts/benchmark.py:212-222, :668-674)."""
    pairs = sum(int(a) * int(b) for a, b in zip(q_lens, kv_lens))
    fwd = 4 * heads * head_dim * pairs
    return {"fwd": fwd, "bwd": fwd * 5 // 2, "fwd_bwd": fwd * 7 // 2}[mode]
