"""MXFP8 inputs (e4m3 elements, one e8m0 scale per 32 elements) for the jagged GDPA forward.

The reference's block-scaled variant takes unpadded e4m3 ``[total, H, D]`` tensors plus scale tensors that are
padded per sequence to a multiple of 128 rows and laid out in 512-byte atoms, with ``cu_seqlens_sf_q`` /
``cu_seqlens_sf_k`` giving the padded row offsets (gdpa/src/interface.py:604-605, :714-750; layouts
gdpa/src/flash_fwd_sm100.py:746-833).  Its producer, ``quantize_varlen_mxfp8_sf_only``, is referred to
(gdpa/src/interface.py:715-724) but is not in its tree.  This module is that producer, the inverse map, and a
forward entry point that takes the format.

The forward de-quantises Q, K and V to bf16 in one HBM-bound pass each (every e4m3 value times a power of two is
a bf16 number, so nothing is rounded) and runs the bf16 kernel: the products of ``Q K^T`` are then exactly those
a block-scaled tensor-core instruction forms, accumulated in fp32 like there, while P stays bf16 instead of
being re-quantised to e4m3 per 32 columns.  Block-scaled ``tcgen05.mma`` is not used.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _cabi
from .ops import _stream_ptr, generalized_dot_product_attention

__all__ = ["quantize_varlen_mxfp8_sf_only", "dequantize_mxfp8", "generalized_dot_product_attention_mxfp8"]


def _check_offsets(x: torch.Tensor, offsets: torch.Tensor) -> None:
    if offsets.dtype not in (torch.int32, torch.int64) or offsets.device != x.device or offsets.dim() != 1:
        raise ValueError("cu_seqlens must be a 1-D int32 / int64 tensor on the device of the data")
    if offsets.numel() < 1:
        raise ValueError("cu_seqlens must hold at least one entry")


def _run(quantize: bool, x: torch.Tensor, x8: torch.Tensor, sf: torch.Tensor, offsets: torch.Tensor,
         scale_axis: int, sf_blocks: int) -> torch.Tensor:
    total, H, D = x.shape
    batch = offsets.numel() - 1
    blk_off = torch.empty(batch + 1, dtype=offsets.dtype, device=x.device)
    p = _cabi.GdpaMxParams()
    p.struct_size = C.sizeof(_cabi.GdpaMxParams)
    p.x_is_fp32 = int(x.dtype == torch.float32)
    p.x, p.x8, p.sf = x.data_ptr(), x8.data_ptr(), sf.data_ptr()
    p.offsets, p.block_offsets = offsets.data_ptr(), blk_off.data_ptr()
    p.offsets_are_int64 = int(offsets.dtype == torch.int64)
    p.batch, p.total, p.heads, p.head_dim = batch, total, H, D
    p.scale_axis, p.sf_blocks = int(scale_axis), int(sf_blocks)
    fn = _cabi.lib.gdpa_quantize_mxfp8 if quantize else _cabi.lib.gdpa_dequantize_mxfp8
    _cabi.check(fn(C.byref(p), _stream_ptr()), "gdpa_quantize_mxfp8" if quantize else "gdpa_dequantize_mxfp8")
    return blk_off


def _sf_shape(H: int, D: int, sf_blocks: int, scale_axis: int) -> Tuple[int, ...]:
    d_atoms = (D + 127) // 128
    return (H, sf_blocks, d_atoms, 32, 4, 4) if scale_axis == 0 else (H, d_atoms, sf_blocks, 32, 4, 4)


def quantize_varlen_mxfp8_sf_only(
    x: torch.Tensor,
    cu_seqlens: torch.Tensor,
    scale_axis: int = 0,
    exact_layout: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantise a jagged ``[total, H, D]`` CUDA tensor (bf16 or fp32) to MXFP8.

    ``scale_axis=0`` puts the 32-element blocks along the head dim (Q and K, contracted over D);
    ``scale_axis=1`` along the tokens of each sequence (V, contracted over the KV tokens).  Returns
    ``(x8, sf, cu_seqlens_sf)``: ``x8`` e4m3 of the shape of ``x`` (only the scales are padded), ``sf`` the
    e8m0 scales as ``[H, blocks, ceil(D/128), 32, 4, 4]`` (axis 0) or ``[H, ceil(D/128), blocks, 32, 4, 4]``
    (axis 1) — element ``[..., r0, r1, k]`` of an atom is the scale of its row ``r0 + 32 * r1`` and 32-element
    block ``k`` — and ``cu_seqlens_sf`` (int32) the 128-aligned row offsets of the sequences in the padded scale
    rows.  With ``exact_layout`` the number of blocks is exactly that of the batch, as the reference lays its
    scale tensors out (one read of the sequence lengths on the host); without it, the upper bound
    ``total // 128 + batch`` is used and nothing synchronises.
    """
    if not x.is_cuda or x.dim() != 3 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("quantize_varlen_mxfp8_sf_only expects a CUDA [total, H, D] tensor of bf16 or fp32")
    if scale_axis not in (0, 1):
        raise ValueError("scale_axis must be 0 (head dim) or 1 (tokens)")
    if x.shape[2] % 32 != 0:
        raise ValueError("head_dim must be a multiple of 32")
    _check_offsets(x, cu_seqlens)
    x = x.contiguous()
    cu_seqlens = cu_seqlens.contiguous()
    total, H, D = x.shape
    batch = cu_seqlens.numel() - 1
    if exact_layout:
        lens = torch.diff(cu_seqlens.to("cpu", torch.int64)).clamp_min(0)
        sf_blocks = int(((lens + 127) // 128).sum())
    else:
        sf_blocks = total // 128 + batch
    with torch.cuda.device(x.device):
        x8 = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        sf = torch.zeros(_sf_shape(H, D, max(sf_blocks, 1), scale_axis), dtype=torch.uint8, device=x.device)
        blk_off = _run(True, x, x8, sf, cu_seqlens, scale_axis, max(sf_blocks, 1) if total > 0 else 0)
        cu_sf = (blk_off * 128).to(torch.int32)
    return x8, sf.view(torch.float8_e8m0fnu), cu_sf


def dequantize_mxfp8(
    x8: torch.Tensor,
    sf: torch.Tensor,
    cu_seqlens: torch.Tensor,
    scale_axis: int = 0,
    dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """The values of an MXFP8 tensor (layout of :func:`quantize_varlen_mxfp8_sf_only`) as bf16 (exact) or fp32."""
    if not x8.is_cuda or x8.dim() != 3 or x8.dtype != torch.float8_e4m3fn:
        raise ValueError("dequantize_mxfp8 expects a CUDA [total, H, D] float8_e4m3fn tensor")
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("dtype must be bf16 or fp32")
    if scale_axis not in (0, 1):
        raise ValueError("scale_axis must be 0 (head dim) or 1 (tokens)")
    _check_offsets(x8, cu_seqlens)
    total, H, D = x8.shape
    if D % 32 != 0:
        raise ValueError("head_dim must be a multiple of 32")
    d_atoms = (D + 127) // 128
    if sf.device != x8.device or sf.element_size() != 1 or sf.numel() % (H * d_atoms * 512) != 0:
        raise ValueError("sf must hold whole 512-byte atoms for every head on the device of the data")
    sf_blocks = sf.numel() // (H * d_atoms * 512)
    x8 = x8.contiguous()
    sf = sf.contiguous()
    with torch.cuda.device(x8.device):
        out = torch.empty(x8.shape, dtype=dtype, device=x8.device)
        _run(False, out, x8, sf, cu_seqlens.contiguous(), scale_axis, sf_blocks)
    return out


def generalized_dot_product_attention_mxfp8(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    sfq: torch.Tensor,
    sfk: torch.Tensor,
    sfv: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: Optional[float] = None,
    activation: str = "softmax",
    cu_seqlens_sf_q: Optional[torch.Tensor] = None,
    cu_seqlens_sf_k: Optional[torch.Tensor] = None,
    window_size: Optional[int] = None,
) -> torch.Tensor:
    """Forward for MXFP8 Q, K (scales along the head dim) and V (scales along the tokens); bf16 output, as the
    reference's low-precision forward returns (gdpa/src/interface.py:1053).  ``cu_seqlens_sf_q`` /
    ``cu_seqlens_sf_k`` are implied by the offsets (128-aligned prefix sums); when given they are checked for
    length only.  Forward only: no gradients flow to the quantised inputs."""
    for name, cu, off in (("cu_seqlens_sf_q", cu_seqlens_sf_q, query_offset), ("cu_seqlens_sf_k", cu_seqlens_sf_k, key_offset)):
        if cu is not None and cu.numel() != off.numel():
            raise ValueError(f"{name} must have one entry per offset")
    with torch.no_grad():
        q = dequantize_mxfp8(query, sfq, query_offset, 0)
        k = dequantize_mxfp8(key, sfk, key_offset, 0)
        v = dequantize_mxfp8(value, sfv, key_offset, 1)
        return generalized_dot_product_attention(q, k, v, query_offset, key_offset, int(max_seq_len_q), int(max_seq_len_kv),
                                                 qk_scale=qk_scale, activation=activation, window_size=window_size)
