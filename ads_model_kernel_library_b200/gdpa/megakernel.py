"""GDPA with the norms either side of it: ``LayerNorm(Q) -> GDPA -> + Q residual -> RMSNorm -> + residual``.

Host side of the reference's ``tlx_gdpa_megakernel`` entry point
(gdpa_megakernel/src/tlx_gdpa_megakernel.py:8155-8192), forward and backward.  Both norms run over all
``heads * head_dim`` values of a token (eps 1e-5, :402 and :481).  Here the pipeline is three launches of
libgdpa_b200.so: ``gdpa_layernorm_rows`` writes the normalised Q, ``gdpa_fwd`` adds the Q residual and
accumulates every row's sum of squares in its epilogue, ``gdpa_rmsnorm_rows`` scales the rows in place
(and adds the generic residual).  The reference does the same in one launch with a cluster of one CTA per
head; the order of operations is the same (:1076-1142): the Q residual goes in before the RMS norm, the
generic residual after it.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch

from . import _cabi
from .math import SOFTMAX_ID, activation_string_to_int
from .ops import (_build_schedule, _check_inputs, _fill_fwd_params, _set_timing, _stream_ptr, expect_contiguous)

NORM_EPS = 1e-5


def _norm_params(x: torch.Tensor, out: torch.Tensor, n: int, eps: float) -> _cabi.GdpaNormParams:
    p = _cabi.GdpaNormParams()
    p.struct_size = C.sizeof(_cabi.GdpaNormParams)
    p.n = n
    p.rows = x.shape[0]
    p.x = x.data_ptr()
    p.out = out.data_ptr()
    p.eps = eps
    return p


def _vector(t: Optional[torch.Tensor], n: int, name: str, device) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.numel() != n or t.device != device:
        raise ValueError(f"{name} must hold heads * head_dim = {n} values on the device of query")
    return t.detach().reshape(n).to(torch.float32).contiguous()


def layernorm_rows(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                   eps: float = NORM_EPS, stats: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """Layer norm of every token row of a contiguous bf16 ``[T, H, D]`` tensor over its ``H * D`` values.
    ``stats = (mean, rstd)``: optional fp32 ``[T]`` tensors that receive the row statistics (for the backward)."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
        raise ValueError("layernorm_rows expects a contiguous bf16 CUDA tensor")
    n = int(torch.Size(x.shape[1:]).numel())
    out = torch.empty_like(x)
    w, b = _vector(weight, n, "layernorm_weight", x.device), _vector(bias, n, "layernorm_bias", x.device)
    with torch.cuda.device(x.device):
        p = _norm_params(x, out, n, eps)
        p.weight = w.data_ptr() if w is not None else None
        p.bias = b.data_ptr() if b is not None else None
        if stats is not None:
            p.row_mean, p.row_rstd = stats[0].data_ptr(), stats[1].data_ptr()
        _cabi.check(_cabi.lib.gdpa_layernorm_rows(C.byref(p), _stream_ptr()), "gdpa_layernorm_rows")
    return out


def rmsnorm_rows(x: torch.Tensor, weight: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 row_sumsq: Optional[torch.Tensor] = None, eps: float = NORM_EPS, out: Optional[torch.Tensor] = None,
                 row_rstd: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of every token row over ``H * D`` values, times ``weight``, plus ``residual``; ``row_sumsq``
    are the rows' sums of squares when the producer of ``x`` already has them."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
        raise ValueError("rmsnorm_rows expects a contiguous bf16 CUDA tensor")
    n = int(torch.Size(x.shape[1:]).numel())
    out = torch.empty_like(x) if out is None else out
    w = _vector(weight, n, "rms_norm_weight", x.device)
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise ValueError("residual must be a contiguous tensor of the shape and dtype of the output")
    with torch.cuda.device(x.device):
        p = _norm_params(x, out, n, eps)
        p.weight = w.data_ptr() if w is not None else None
        p.residual = residual.data_ptr() if residual is not None else None
        p.row_sumsq = row_sumsq.data_ptr() if row_sumsq is not None else None
        p.row_rstd = row_rstd.data_ptr() if row_rstd is not None else None
        _cabi.check(_cabi.lib.gdpa_rmsnorm_rows(C.byref(p), _stream_ptr()), "gdpa_rmsnorm_rows")
    return out


def norm_rows_backward(mode: int, dy: torch.Tensor, dy_add: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
                       weight: Optional[torch.Tensor] = None, row_mean: Optional[torch.Tensor] = None,
                       row_rstd: Optional[torch.Tensor] = None, want_dweight: bool = False, want_dbias: bool = False):
    """Backward of a row norm (``mode`` 0 = RMS norm, 1 = layer norm, 2 = plain sum ``dy + dy_add``):
    returns ``(dx, dweight, dbias)`` with the last two ``None`` unless asked for."""
    n = int(torch.Size(dy.shape[1:]).numel())
    dx = torch.empty_like(dy)
    w = _vector(weight, n, "weight", dy.device)
    dw = torch.zeros(n, dtype=torch.float32, device=dy.device) if want_dweight else None
    db = torch.zeros(n, dtype=torch.float32, device=dy.device) if want_dbias else None
    with torch.cuda.device(dy.device):
        p = _cabi.GdpaNormBwdParams()
        p.struct_size = C.sizeof(_cabi.GdpaNormBwdParams)
        p.mode, p.rows, p.n = mode, dy.shape[0], n
        p.dy, p.dx = dy.data_ptr(), dx.data_ptr()
        p.dy_add = dy_add.data_ptr() if dy_add is not None else None
        p.x = x.data_ptr() if x is not None else None
        p.weight = w.data_ptr() if w is not None else None
        p.row_mean = row_mean.data_ptr() if row_mean is not None else None
        p.row_rstd = row_rstd.data_ptr() if row_rstd is not None else None
        p.dweight = dw.data_ptr() if dw is not None else None
        p.dbias = db.data_ptr() if db is not None else None
        _cabi.check(_cabi.lib.gdpa_norm_rows_bwd(C.byref(p), _stream_ptr()), "gdpa_norm_rows_bwd")
    return dx, dw, db


@torch.library.custom_op("gdpa::gdpa_with_norms", mutates_args=(), device_types="cuda")
def _gdpa_with_norms_op(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    activation: int,
    window_size: int,
    fused_layernorm: bool,
    layernorm_weight: Optional[torch.Tensor],
    layernorm_bias: Optional[torch.Tensor],
    fused_q_residual_add: bool,
    fused_rms_norm: bool,
    rms_norm_weight: Optional[torch.Tensor],
    residual: Optional[torch.Tensor],
    save_for_backward: bool,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(out, x, q_norm, ln_mean, ln_rstd, rrms)``: the result, and what the backward needs — the value
    that entered the RMS norm, the normalised Q and the row statistics of the two norms (empty tensors for what
    does not apply or when ``save_for_backward`` is false)."""
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.bfloat16)
    if not query.is_contiguous():
        raise ValueError("query must be contiguous for the norm pipeline")
    dev, T = query.device, query.shape[0]
    none = lambda dtype=torch.float32: torch.empty(0, dtype=dtype, device=dev)  # noqa: E731
    with torch.cuda.device(dev):
        keep_ln = fused_layernorm and save_for_backward
        ln_mean = torch.empty(T, dtype=torch.float32, device=dev) if keep_ln else none()
        ln_rstd = torch.empty(T, dtype=torch.float32, device=dev) if keep_ln else none()
        q_in = (layernorm_rows(query, layernorm_weight, layernorm_bias, stats=(ln_mean, ln_rstd) if keep_ln else None)
                if fused_layernorm else query)
        o = torch.empty(query.shape, dtype=query.dtype, device=dev)
        keep_rms = fused_rms_norm and save_for_backward
        rrms = torch.empty(T, dtype=torch.float32, device=dev) if keep_rms else none()
        q_norm = q_in if fused_layernorm else none(query.dtype)
        if T == 0 or batch == 0:
            return o, none(query.dtype), q_norm, ln_mean, ln_rstd, rrms
        sumsq = torch.zeros(T, dtype=torch.float32, device=dev) if fused_rms_norm else None
        sched = _build_schedule(_cabi.GDPA_SCHED_FWD, query_offset, key_offset, batch, H, T, max_seq_len_q, max_seq_len_kv)
        p = _fill_fwd_params(q_in, key, value, o, query_offset, key_offset, batch, H, D, max_seq_len_q, max_seq_len_kv,
                             qk_scale, activation, sched, _cabi.GDPA_DTYPE_BF16)
        p.window_plus_one = window_size + 1 if window_size >= 0 else 0
        if fused_q_residual_add:
            p.residual = q_in.data_ptr()
        elif residual is not None and not fused_rms_norm:
            p.residual = residual.data_ptr()  # without a norm in between the generic residual is a plain add
        if sumsq is not None:
            p.row_sumsq = sumsq.data_ptr()
        _set_timing(p, "fwd")
        _cabi.check(_cabi.lib.gdpa_fwd(C.byref(p), _stream_ptr()), "gdpa_fwd")
        if not fused_rms_norm:
            return o, none(query.dtype), q_norm, ln_mean, ln_rstd, rrms
        if keep_rms:  # the backward needs the value that entered the norm: normalise into a second tensor
            out = rmsnorm_rows(o, rms_norm_weight, residual, sumsq, row_rstd=rrms)
            return out, o, q_norm, ln_mean, ln_rstd, rrms
        rmsnorm_rows(o, rms_norm_weight, residual, sumsq, out=o)
    return o, none(query.dtype), q_norm, ln_mean, ln_rstd, rrms


@_gdpa_with_norms_op.register_fake
def _(query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, qk_scale, activation, window_size,
      fused_layernorm, layernorm_weight, layernorm_bias, fused_q_residual_add, fused_rms_norm, rms_norm_weight, residual,
      save_for_backward):
    T = query.shape[0]
    f32 = lambda n: torch.empty(n, dtype=torch.float32, device=query.device)  # noqa: E731
    keep_ln, keep_rms = fused_layernorm and save_for_backward, fused_rms_norm and save_for_backward
    return (query.new_empty(query.shape), query.new_empty(query.shape if keep_rms else (0,)),
            query.new_empty(query.shape if fused_layernorm else (0,)), f32(T if keep_ln else 0), f32(T if keep_ln else 0),
            f32(T if keep_rms else 0))


def _norms_setup_context(ctx, inputs, output):
    (query, key, value, query_offset, key_offset, max_q, max_kv, qk_scale, activation, window, fused_layernorm, ln_w, ln_b,
     fused_q_residual_add, fused_rms_norm, rms_w, residual, saved) = inputs
    _, x, q_norm, ln_mean, ln_rstd, rrms = output
    ctx.save_for_backward(query, key, value, query_offset, key_offset, x, q_norm, ln_mean, ln_rstd, rrms, ln_w, rms_w)
    ctx.cfg = (max_q, max_kv, qk_scale, activation, window, fused_layernorm, fused_q_residual_add, fused_rms_norm,
               ln_b is not None, residual is not None, saved)
    ctx.ln_b_like = ln_b


def _like(grad: Optional[torch.Tensor], ref: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if (grad is None or ref is None) else grad.to(ref.dtype).reshape(ref.shape)


def _norms_backward(ctx, dout, *_unused):
    """Chain rule through the pipeline, each step one launch of the library: RMS-norm backward, the GDPA backward
    with dO = d x, layer-norm backward of (dQ + d x) (the Q residual adds d x to the gradient of the normalised Q)."""
    query, key, value, query_offset, key_offset, x, q_norm, ln_mean, ln_rstd, rrms, ln_w, rms_w = ctx.saved_tensors
    max_q, max_kv, qk_scale, activation, window, f_ln, f_qres, f_rms, has_ln_b, has_res, saved = ctx.cfg
    if not saved:
        raise RuntimeError("gdpa_megakernel was run without saving what its backward needs")
    dout = dout.contiguous()
    d_rms_w = None
    if f_rms:
        d_x, d_rms_w, _ = norm_rows_backward(0, dout, None, x, rms_w, None, rrms, want_dweight=rms_w is not None)
    else:
        d_x = dout
    dq_n, dk, dv = torch.ops.gdpa.generalized_dot_product_attention_backward(
        d_x, q_norm if f_ln else query, key, value, query_offset, key_offset, max_q, max_kv, qk_scale, activation, None, None,
        window)
    d_ln_w = d_ln_b = None
    if f_ln:
        dq, d_ln_w, d_ln_b = norm_rows_backward(1, dq_n, d_x if f_qres else None, query, ln_w, ln_mean, ln_rstd,
                                                want_dweight=ln_w is not None, want_dbias=has_ln_b)
    elif f_qres:
        dq = norm_rows_backward(2, dq_n, d_x)[0]
    else:
        dq = dq_n
    return (dq, dk, dv, None, None, None, None, None, None, None, None, _like(d_ln_w, ln_w), _like(d_ln_b, ctx.ln_b_like), None,
            None, _like(d_rms_w, rms_w), dout if has_res else None, None)


_gdpa_with_norms_op.register_autograd(_norms_backward, setup_context=_norms_setup_context)


def gdpa_megakernel(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    ad_to_request_offset: Optional[torch.Tensor] = None,
    attn_mask: Optional[torch.Tensor] = None,
    attn_offset: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    qk_scale: Optional[float] = None,
    seq_index: Optional[torch.Tensor] = None,
    allow_tf32: bool = True,
    output_offset: Optional[torch.Tensor] = None,
    use_start_end_offsets: bool = False,
    window_size: Optional[int] = None,
    broadcast_q: bool = False,
    activation: str = "fast_gelu",
    enable_persistent: bool = False,
    enable_tma: bool = False,
    enable_ws: bool = False,
    use_dq_atomic_add: bool = False,
    total_num_objects: Optional[int] = None,
    bwd_opt_tech: str = "base",
    cpu_query_offset: Optional[torch.Tensor] = None,
    use_on_device_tma: bool = False,
    ensemble_activation_list: Optional[List[int]] = None,
    fused_rms_norm: bool = False,
    rms_norm_weight: Optional[torch.Tensor] = None,
    fused_residual_add: bool = False,
    residual: Optional[torch.Tensor] = None,
    fused_q_residual_add: bool = False,
    fused_layernorm: bool = False,
    layernorm_weight: Optional[torch.Tensor] = None,
    layernorm_bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Same signature as the reference's ``tlx_gdpa_megakernel``; forward and backward.

    ``out = RMSNorm(GDPA(q', K, V) + q') * rms_norm_weight + residual`` with ``q' = LayerNorm(query)`` when
    ``fused_layernorm`` (else ``query``), the ``+ q'`` only with ``fused_q_residual_add``, the norm only with
    ``fused_rms_norm``, the ``+ residual`` only with ``fused_residual_add``.  Scheduling options are
    accepted and ignored; masks, causality, start/end offsets, ``broadcast_q``, ``ad_to_request_offset`` and
    activation ensembles raise ``NotImplementedError`` here."""
    if attn_mask is not None or is_causal:
        raise NotImplementedError("attn_mask / is_causal unsupported")
    if (attn_offset is not None or output_offset is not None or use_start_end_offsets or broadcast_q
            or ad_to_request_offset is not None or ensemble_activation_list):
        raise NotImplementedError("this option is not supported together with the fused norms")
    if fused_layernorm and not fused_rms_norm:
        raise ValueError("fused_layernorm requires fused_rms_norm")  # the reference asserts the same (:4441-4444)
    if fused_residual_add and residual is None:
        raise ValueError("fused_residual_add needs the residual tensor")
    if fused_residual_add and fused_q_residual_add and not fused_rms_norm:
        raise NotImplementedError("two residuals without a norm between them are not supported")
    act_id = activation_string_to_int(activation)
    if act_id == SOFTMAX_ID:
        raise NotImplementedError("the fused norms are built for the element-wise activations")
    scale = 1.0 if qk_scale is None else float(qk_scale)
    window = -1 if window_size is None else int(window_size)
    res = expect_contiguous(residual) if fused_residual_add else None
    if res is not None and (res.shape != query.shape or res.dtype != query.dtype):
        raise ValueError("residual must have the shape and dtype of query")
    ln_w, ln_b = (layernorm_weight, layernorm_bias) if fused_layernorm else (None, None)
    rms_w = rms_norm_weight if fused_rms_norm else None
    save = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (query, key, value, ln_w, ln_b, rms_w, res))
    return torch.ops.gdpa.gdpa_with_norms(
        expect_contiguous(query), expect_contiguous(key), expect_contiguous(value), query_offset, key_offset,
        int(max_seq_len_q), int(max_seq_len_kv), scale, act_id, window, bool(fused_layernorm), ln_w, ln_b,
        bool(fused_q_residual_add), bool(fused_rms_norm), rms_w, res, save)[0]


tlx_gdpa_megakernel = gdpa_megakernel
