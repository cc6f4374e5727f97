"""Host side of the GDPA operator: the reference's Python entry point, re-implemented over the
C-ABI kernel library.

``generalized_dot_product_attention`` keeps the name, the positional order and the keyword
names of the reference function (gdpa/triton/triton_generalized_dot_product_attention.py:4229-4267)
and is backed by the torch custom op ``gdpa::generalized_dot_product_attention`` with autograd
registered the same way the reference does it (:3099, :3888-3894).  PyTorch is used for device
memory and streams only; all arithmetic runs in libgdpa_b200.so.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

import torch

from . import _cabi
from .math import SOFTMAX_ID, activation_string_to_int, int_to_activation

_SUPPORTED_HEAD_DIMS = (64, 128)
_status_words = {}
_timing_events = {"fwd": None, "bwd": None}


class kernel_timing:
    """Context manager for benchmarks: record a pair of ``torch.cuda.Event`` (``enable_timing=True``)
    immediately around the main forward and/or backward kernel of every operator call made inside
    the block, so that the kernel can be timed without the schedule build, the accumulator memset
    and the dQ rounding pass."""

    def __init__(self, fwd=None, bwd=None):
        self.new = {"fwd": fwd, "bwd": bwd}

    def __enter__(self):
        self.old = dict(_timing_events)
        for pair in self.new.values():
            if pair is not None:
                for ev in pair:  # events are created lazily by their first record
                    ev.record()
        _timing_events.update(self.new)
        return self

    def __exit__(self, *exc):
        _timing_events.update(self.old)
        return False


def _set_timing(p, which: str) -> None:
    pair = _timing_events[which]
    if pair is not None:
        p.timing_start_event = pair[0].cuda_event
        p.timing_stop_event = pair[1].cuda_event


_ROLE_NAMES = {1: "TMA loader", 2: "MMA issuer", 3: "activation warps", 4: "epilogue", 5: "dQ reduce warps", 6: "tail fixer"}


def _device_key(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the kernels write when one of their bounded waits runs out.  It lives in pinned host
    memory, which the device addresses directly (unified addressing), so the host can look at it at any time
    without synchronising; the kernels touch it only on that failure path."""
    key = _device_key(device)
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[key] = t
    return t


def _describe_status(code: int) -> str:
    return (f"a kernel wait ran out (status 0x{code:x}: barrier {code >> 8}, role {_ROLE_NAMES.get(code & 0xff, code & 0xff)}); "
            "results of the calls since the last check on this device are incomplete")


def _raise_if_wait_ran_out(device: torch.device) -> None:
    """Called at the start of every operator call: if a kernel of an EARLIER call on this device gave up on a wait,
    raise now (and clear the word).  A plain host read, no synchronisation."""
    t = _status_words.get(_device_key(device))
    if t is not None:
        code = int(t[0])
        if code != 0:
            t.zero_()
            raise RuntimeError(_describe_status(code))


def kernel_status(device=None) -> int:
    """Synchronise the device, then read (and clear) its status word: 0 = every wait of every kernel launched so
    far completed.  For tests and diagnostics; the operator itself checks the word, without synchronising, at the
    start of the next call on the device."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status_word(device)
    torch.cuda.synchronize(device)
    v = int(t[0])
    if v != 0:
        t.zero_()
    return v


_validate_offsets = os.environ.get("GDPA_CHECK_OFFSETS", "0") not in ("", "0")


def set_offset_validation(enabled: bool) -> bool:
    """Switch the host-side check of the offset arrays on or off (default: the environment variable
    ``GDPA_CHECK_OFFSETS=1``, else off); returns the previous setting.  When on, every operator call copies its
    offset arrays to the host (a synchronisation) and raises ``ValueError`` before anything is launched if they are
    not non-negative, non-decreasing and inside the tensors.  When off the arrays are trusted, as the reference
    trusts them; the kernels then only guarantee that they do not access memory outside the tensors."""
    global _validate_offsets
    old, _validate_offsets = _validate_offsets, bool(enabled)
    return old


def _check_offsets(name: str, off: torch.Tensor, rows: int, start_end: bool) -> None:
    o = off.detach().to("cpu", torch.int64)
    if o.numel() == 0:
        return
    if int(o.min()) < 0 or int(o.max()) > rows:
        raise ValueError(f"{name} has entries outside [0, {rows}] (the rows of its tensor)")
    if start_end:
        if bool((o[1::2] < o[0::2]).any()):
            raise ValueError(f"{name} holds a [start, end] pair with end < start")
    elif bool((o[1:] < o[:-1]).any()):
        raise ValueError(f"{name} must be non-decreasing (exclusive prefix sums of the sequence lengths)")


def _maybe_validate(qo, ko, total_q: int, total_kv: int, start_end: bool = False, kv_index=None) -> None:
    if not _validate_offsets:
        return
    _check_offsets("query_offset", qo, total_q, start_end)
    _check_offsets("key_offset", ko, total_kv, start_end)
    if kv_index is not None and kv_index.numel() > 0:
        idx = kv_index.detach().to("cpu", torch.int64)
        if int(idx.min()) < 0 or int(idx.max()) >= ko.numel() - 1:
            raise ValueError("ad_to_request_offset has entries outside [0, number of KV sequences)")


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_inputs(q, k, v, qo, ko, dtype, shared_kv: bool = False, start_end: bool = False) -> Tuple[int, int, int]:
    if q.is_cuda:
        _raise_if_wait_ran_out(q.device)
    for name, t in (("query", q), ("key", k), ("value", v)):
        if t.dim() != 3:
            raise ValueError(f"{name} must be [total_tokens, H, D], got {tuple(t.shape)}")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: this operator has no CPU path")
        if t.dtype != dtype:
            raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
        if t.stride(2) != 1 or (t.stride(1) * t.element_size()) % 16 or (t.stride(0) * t.element_size()) % 16 \
                or t.stride(1) < t.shape[2] or t.stride(0) < t.stride(1) * t.shape[1] or t.data_ptr() % 16:
            raise ValueError(f"{name} must have a contiguous head dimension and 16-byte aligned row / head strides "
                             "(a contiguous tensor, or a slice of a packed QKV / KV tensor along the last dimension)")
    if k.shape != v.shape:
        raise ValueError("key and value must have the same shape")
    H, D = q.shape[1], q.shape[2]
    if k.shape[2] != D:
        raise NotImplementedError("query and key/value must have the same head_dim")
    if k.shape[1] < 1 or H % k.shape[1] != 0:
        raise ValueError("the number of query heads must be a multiple of the number of key/value heads")
    if D not in _SUPPORTED_HEAD_DIMS:
        raise NotImplementedError(f"head_dim {D} is not supported (supported: {_SUPPORTED_HEAD_DIMS})")
    for name, t in (("query_offset", qo), ("key_offset", ko)):
        if t.dim() != 1 or t.numel() < 1:
            raise ValueError(f"{name} must be a 1-D tensor of batch + 1 entries")
        if t.dtype not in (torch.int32, torch.int64):
            raise TypeError(f"{name} must be int32 or int64, got {t.dtype}")
        if t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as query")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if qo.dtype != ko.dtype or (qo.numel() != ko.numel() and not shared_kv):
        raise ValueError("query_offset and key_offset must have the same length and dtype")
    if start_end and qo.numel() % 2 != 0:
        raise ValueError("start / end offsets hold two entries per sequence")
    _maybe_validate(qo, ko, q.shape[0], k.shape[0], start_end)
    if start_end:
        return qo.numel() // 2, H, D
    return qo.numel() - 1, H, D


def _offset_flags(offsets: torch.Tensor, start_end: bool = False) -> int:
    return (_cabi.GDPA_OFFSETS_INT64 if offsets.dtype == torch.int64 else 0) | (_cabi.GDPA_OFFSETS_PAIRS if start_end else 0)


def _build_schedule(mode: int, qo, ko, batch: int, heads: int, total_rows: int, max_q: int, max_kv: int,
                    kv_index: Optional[torch.Tensor] = None, start_end: bool = False) -> torch.Tensor:
    nbytes = _cabi.lib.gdpa_schedule_bytes(mode, total_rows, batch, heads)
    sched = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=qo.device)
    p = _cabi.GdpaSchedParams()
    p.struct_size = C.sizeof(_cabi.GdpaSchedParams)
    p.mode = mode
    p.q_offsets = qo.data_ptr()
    p.kv_offsets = ko.data_ptr()
    p.offsets_are_int64 = _offset_flags(qo, start_end)
    p.batch = batch
    p.heads = heads
    p.max_seq_len_q = max_q
    p.max_seq_len_kv = max_kv
    p.schedule = sched.data_ptr()
    p.schedule_bytes = sched.numel() * 4
    if kv_index is not None:
        p.kv_seq_index = kv_index.data_ptr()
        p.kv_batch = ko.numel() - 1
    _cabi.check(_cabi.lib.gdpa_build_schedule(C.byref(p), _stream_ptr()), "gdpa_build_schedule")
    return sched


def _fill_fwd_params(q, k, v, o, qo, ko, batch, H, D, max_q, max_kv, scale, act_id, sched, dtype_id) -> _cabi.GdpaFwdParams:
    p = _cabi.GdpaFwdParams()
    p.struct_size = C.sizeof(_cabi.GdpaFwdParams)
    p.dtype = dtype_id
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.q_offsets, p.kv_offsets = qo.data_ptr(), ko.data_ptr()
    p.offsets_are_int64 = int(qo.dtype == torch.int64)
    p.batch = batch
    p.total_q, p.total_kv = q.shape[0], k.shape[0]
    p.heads, p.head_dim = H, D
    for field, t in (("q_strides", q), ("k_strides", k), ("v_strides", v)):
        getattr(p, field)[0], getattr(p, field)[1] = t.stride(0), t.stride(1)
    p.kv_heads = k.shape[1]  # grouped-query attention when smaller than H
    p.max_seq_len_q, p.max_seq_len_kv = max_q, max_kv
    p.activation = act_id
    p.qk_scale = scale
    p.schedule = sched.data_ptr()
    p.status = _status_word(q.device).data_ptr()
    return p


@torch.library.custom_op("gdpa::generalized_dot_product_attention", mutates_args=(), device_types="cuda")
def _gdpa_forward_op(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    activation: int,
    window_size: int = -1,
    start_end_offsets: bool = False,
) -> torch.Tensor:
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.bfloat16, start_end=start_end_offsets)
    with torch.cuda.device(query.device):
        o = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        if query.shape[0] == 0 or batch == 0:
            return o
        # with start / end offsets the longest sequence is not bounded by the rows of the tensors
        sched = _build_schedule(_cabi.GDPA_SCHED_FWD, query_offset, key_offset, batch, H,
                                batch * max_seq_len_q if start_end_offsets else query.shape[0],
                                max_seq_len_q, max_seq_len_kv, start_end=start_end_offsets)
        p = _fill_fwd_params(query, key, value, o, query_offset, key_offset, batch, H, D, max_seq_len_q,
                             max_seq_len_kv, qk_scale, activation, sched, _cabi.GDPA_DTYPE_BF16)
        p.offsets_are_int64 = _offset_flags(query_offset, start_end_offsets)
        p.window_plus_one = window_size + 1 if window_size >= 0 else 0
        _set_timing(p, "fwd")
        _cabi.check(_cabi.lib.gdpa_fwd(C.byref(p), _stream_ptr()), "gdpa_fwd")
    return o


@_gdpa_forward_op.register_fake
def _(query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, qk_scale, activation, window_size=-1,
      start_end_offsets=False):
    return query.new_empty(query.shape)


@torch.library.custom_op("gdpa::generalized_dot_product_attention_backward", mutates_args=(), device_types="cuda")
def _gdpa_backward_op(
    do: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    activation: int,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    window_size: int = -1,
    start_end_offsets: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.bfloat16, start_end=start_end_offsets)
    if activation == SOFTMAX_ID and (out is None or lse is None):
        raise ValueError("the softmax backward needs the forward output and its log-sum-exp")
    if do.shape != query.shape or do.dtype != query.dtype:
        raise ValueError("grad_output must have the shape and dtype of query")
    do = do.contiguous()
    with torch.cuda.device(query.device):
        dq = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        dk = torch.empty(key.shape, dtype=key.dtype, device=key.device)
        dv = torch.empty(value.shape, dtype=value.dtype, device=value.device)
        if batch == 0 or (query.shape[0] == 0 and key.shape[0] == 0):
            return dq, dk, dv
        # backward work items are (sequence, K/V head, KV tile); with grouped-query attention one item
        # walks the Q tiles of every query head of its group
        sched = _build_schedule(_cabi.GDPA_SCHED_BWD, query_offset, key_offset, batch, key.shape[1],
                                batch * max_seq_len_kv if start_end_offsets else key.shape[0],
                                max_seq_len_q, max_seq_len_kv, start_end=start_end_offsets)
        acc_bytes = _cabi.lib.gdpa_bwd_workspace_bytes(query.shape[0], H, D)
        dq_accum = torch.empty(max(acc_bytes // 4, 1), dtype=torch.float32, device=query.device)
        p = _cabi.GdpaBwdParams()
        p.struct_size = C.sizeof(_cabi.GdpaBwdParams)
        p.dtype = _cabi.GDPA_DTYPE_BF16
        p.q, p.k, p.v, p.d_o = query.data_ptr(), key.data_ptr(), value.data_ptr(), do.data_ptr()
        p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        p.q_offsets, p.kv_offsets = query_offset.data_ptr(), key_offset.data_ptr()
        p.offsets_are_int64 = _offset_flags(query_offset, start_end_offsets)
        p.batch = batch
        p.total_q, p.total_kv = query.shape[0], key.shape[0]
        p.heads, p.head_dim = H, D
        for field, t in (("q_strides", query), ("k_strides", key), ("v_strides", value)):
            getattr(p, field)[0], getattr(p, field)[1] = t.stride(0), t.stride(1)
        p.kv_heads = key.shape[1]
        if start_end_offsets:  # K / V rows may belong to several sequences: dK, dV are summed in fp32
            dkv_accum = torch.empty(max(2 * key.numel(), 1), dtype=torch.float32, device=query.device)
            p.dkv_accum = dkv_accum.data_ptr()
        p.max_seq_len_q, p.max_seq_len_kv = max_seq_len_q, max_seq_len_kv
        p.activation = activation
        p.qk_scale = qk_scale
        p.schedule = sched.data_ptr()
        p.dq_accum = dq_accum.data_ptr()
        p.status = _status_word(query.device).data_ptr()
        p.window_plus_one = window_size + 1 if window_size >= 0 else 0
        if activation == SOFTMAX_ID:
            dpsum = torch.empty(max(query.shape[0] * H, 1), dtype=torch.float32, device=query.device)
            out = out.contiguous()
            p.o, p.lse, p.dpsum = out.data_ptr(), lse.data_ptr(), dpsum.data_ptr()
        _set_timing(p, "bwd")
        _cabi.check(_cabi.lib.gdpa_bwd(C.byref(p), _stream_ptr()), "gdpa_bwd")
    return dq, dk, dv


@_gdpa_backward_op.register_fake
def _(do, query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, qk_scale, activation, out=None,
      lse=None, window_size=-1, start_end_offsets=False):
    return query.new_empty(query.shape), key.new_empty(key.shape), value.new_empty(value.shape)


def _setup_context(ctx, inputs, output):
    query, key, value, query_offset, key_offset, max_q, max_kv, qk_scale, activation, window_size, start_end = inputs
    ctx.save_for_backward(query, key, value, query_offset, key_offset)
    ctx.max_q, ctx.max_kv, ctx.qk_scale, ctx.activation, ctx.window_size = max_q, max_kv, qk_scale, activation, window_size
    ctx.start_end = start_end


def _backward(ctx, do):
    query, key, value, query_offset, key_offset = ctx.saved_tensors
    dq, dk, dv = torch.ops.gdpa.generalized_dot_product_attention_backward(
        do, query, key, value, query_offset, key_offset, ctx.max_q, ctx.max_kv, ctx.qk_scale, ctx.activation,
        None, None, ctx.window_size, ctx.start_end
    )
    return dq, dk, dv, None, None, None, None, None, None, None, None


_gdpa_forward_op.register_autograd(_backward, setup_context=_setup_context)


@torch.library.custom_op("gdpa::generalized_dot_product_attention_softmax", mutates_args=(), device_types="cuda")
def _gdpa_forward_softmax_op(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    window_size: int = -1,
    start_end_offsets: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax forward that also returns the base-2 log-sum-exp ``[H, total_q]`` its backward needs."""
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.bfloat16, start_end=start_end_offsets)
    with torch.cuda.device(query.device):
        o = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        lse = torch.zeros((H, query.shape[0]), dtype=torch.float32, device=query.device)
        if query.shape[0] == 0 or batch == 0:
            return o, lse
        sched = _build_schedule(_cabi.GDPA_SCHED_FWD, query_offset, key_offset, batch, H,
                                batch * max_seq_len_q if start_end_offsets else query.shape[0],
                                max_seq_len_q, max_seq_len_kv, start_end=start_end_offsets)
        p = _fill_fwd_params(query, key, value, o, query_offset, key_offset, batch, H, D, max_seq_len_q,
                             max_seq_len_kv, qk_scale, SOFTMAX_ID, sched, _cabi.GDPA_DTYPE_BF16)
        p.offsets_are_int64 = _offset_flags(query_offset, start_end_offsets)
        p.lse = lse.data_ptr()
        p.window_plus_one = window_size + 1 if window_size >= 0 else 0
        _set_timing(p, "fwd")
        _cabi.check(_cabi.lib.gdpa_fwd(C.byref(p), _stream_ptr()), "gdpa_fwd")
    return o, lse


@_gdpa_forward_softmax_op.register_fake
def _(query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, qk_scale, window_size=-1,
      start_end_offsets=False):
    return query.new_empty(query.shape), torch.empty((query.shape[1], query.shape[0]), dtype=torch.float32, device=query.device)


def _softmax_setup_context(ctx, inputs, output):
    query, key, value, query_offset, key_offset, max_q, max_kv, qk_scale, window_size, start_end = inputs
    o, lse = output
    ctx.save_for_backward(query, key, value, query_offset, key_offset, o, lse)
    ctx.max_q, ctx.max_kv, ctx.qk_scale, ctx.window_size, ctx.start_end = max_q, max_kv, qk_scale, window_size, start_end


def _softmax_backward(ctx, do, dlse):
    query, key, value, query_offset, key_offset, o, lse = ctx.saved_tensors
    dq, dk, dv = torch.ops.gdpa.generalized_dot_product_attention_backward(
        do, query, key, value, query_offset, key_offset, ctx.max_q, ctx.max_kv, ctx.qk_scale, SOFTMAX_ID, o, lse,
        ctx.window_size, ctx.start_end
    )
    return dq, dk, dv, None, None, None, None, None, None, None


_gdpa_forward_softmax_op.register_autograd(_softmax_backward, setup_context=_softmax_setup_context)


@torch.library.custom_op("gdpa::generalized_dot_product_attention_shared_kv", mutates_args=(), device_types="cuda")
def _gdpa_forward_shared_kv_op(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    kv_seq_index: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    activation: int,
    window_size: int = -1,
) -> torch.Tensor:
    """Forward where Q sequence i attends to KV sequence ``kv_seq_index[i]`` (the reference's
    ``ad_to_request_offset`` inference path, where many ads share the KV of one request)."""
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.bfloat16, shared_kv=True)
    if kv_seq_index.numel() != batch or kv_seq_index.device != query.device:
        raise ValueError("ad_to_request_offset must hold one KV sequence index per Q sequence, on the device of query")
    kv_index = kv_seq_index.to(query_offset.dtype).contiguous()
    _maybe_validate(query_offset, key_offset, query.shape[0], key.shape[0], kv_index=kv_index)
    with torch.cuda.device(query.device):
        o = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        if query.shape[0] == 0 or batch == 0:
            return o
        sched = _build_schedule(_cabi.GDPA_SCHED_FWD, query_offset, key_offset, batch, H, query.shape[0],
                                max_seq_len_q, max_seq_len_kv, kv_index)
        p = _fill_fwd_params(query, key, value, o, query_offset, key_offset, batch, H, D, max_seq_len_q,
                             max_seq_len_kv, qk_scale, activation, sched, _cabi.GDPA_DTYPE_BF16)
        p.kv_seq_index = kv_index.data_ptr()
        p.kv_batch = key_offset.numel() - 1
        p.window_plus_one = window_size + 1 if window_size >= 0 else 0
        _set_timing(p, "fwd")
        _cabi.check(_cabi.lib.gdpa_fwd(C.byref(p), _stream_ptr()), "gdpa_fwd")
    return o


@_gdpa_forward_shared_kv_op.register_fake
def _(query, key, value, query_offset, key_offset, kv_seq_index, max_seq_len_q, max_seq_len_kv, qk_scale, activation,
      window_size=-1):
    return query.new_empty(query.shape)


def _shared_kv_backward(ctx, do):
    raise NotImplementedError("ad_to_request_offset is an inference path: it has no backward")


_gdpa_forward_shared_kv_op.register_autograd(_shared_kv_backward, setup_context=lambda ctx, inputs, output: None)


@torch.library.custom_op("gdpa::generalized_dot_product_attention_fp8", mutates_args=(), device_types="cuda")
def _gdpa_forward_fp8_op(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    q_scales: torch.Tensor,
    k_scales: torch.Tensor,
    v_scales: torch.Tensor,
    q_block_offsets: torch.Tensor,
    kv_block_offsets: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: float,
    activation: int,
) -> torch.Tensor:
    batch, H, D = _check_inputs(query, key, value, query_offset, key_offset, torch.float8_e4m3fn)
    for name, t in (("q_scales", q_scales), ("k_scales", k_scales), ("v_scales", v_scales)):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.device != query.device:
            raise ValueError(f"{name} must be a contiguous fp32 tensor on the device of query")
    for name, t in (("q_block_offsets", q_block_offsets), ("kv_block_offsets", kv_block_offsets)):
        if t.dtype != query_offset.dtype or t.numel() != batch + 1 or t.device != query.device:
            raise ValueError(f"{name} must have the dtype and length of the offsets")
    with torch.cuda.device(query.device):
        o = torch.empty(query.shape, dtype=torch.bfloat16, device=query.device)
        if query.shape[0] == 0 or batch == 0:
            return o
        sched = _build_schedule(_cabi.GDPA_SCHED_FWD, query_offset, key_offset, batch, H, query.shape[0],
                                max_seq_len_q, max_seq_len_kv)
        p = _fill_fwd_params(query, key, value, o, query_offset, key_offset, batch, H, D, max_seq_len_q,
                             max_seq_len_kv, qk_scale, activation, sched, _cabi.GDPA_DTYPE_FP8_E4M3)
        p.q_scales, p.k_scales, p.v_scales = q_scales.data_ptr(), k_scales.data_ptr(), v_scales.data_ptr()
        p.q_block_offsets, p.kv_block_offsets = q_block_offsets.data_ptr(), kv_block_offsets.data_ptr()
        _set_timing(p, "fwd")
        _cabi.check(_cabi.lib.gdpa_fwd_fp8(C.byref(p), _stream_ptr()), "gdpa_fwd_fp8")
    return o


@_gdpa_forward_fp8_op.register_fake
def _(query, key, value, q_scales, k_scales, v_scales, q_block_offsets, kv_block_offsets, query_offset, key_offset,
      max_seq_len_q, max_seq_len_kv, qk_scale, activation):
    return torch.empty(query.shape, dtype=torch.bfloat16, device=query.device)


def expect_contiguous(x: torch.Tensor) -> torch.Tensor:
    """Same helper as the reference (gdpa/triton/triton_generalized_dot_product_attention.py:4296)."""
    return x if x.is_contiguous() else x.contiguous()


@torch.fx.wrap
def generalized_dot_product_attention(
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
    activation: str = "raw",
    enable_persistent: bool = False,
    enable_tma: bool = False,
    enable_ws: bool = False,
    use_dq_atomic_add: bool = False,
    total_num_objects: Optional[int] = None,
    ts_encoding_params: Optional[torch.Tensor] = None,
    ts_event_request_even_params: Optional[torch.Tensor] = None,
    ts_event_request_log_params: Optional[torch.Tensor] = None,
    ts_adjacent_event_log_params: Optional[torch.Tensor] = None,
    ts_encoding_bucket_values: Optional[torch.Tensor] = None,
    ts_event_request_even_bucket_values: Optional[torch.Tensor] = None,
    ts_event_request_log_bucket_values: Optional[torch.Tensor] = None,
    ts_adjacent_event_log_bucket_values: Optional[torch.Tensor] = None,
    pos_emb_params: Optional[torch.Tensor] = None,
    pos_emb_bucket_values: Optional[torch.Tensor] = None,
    bwd_opt_tech: str = "base",
    ensemble_activation_list: Optional[List[int]] = None,
) -> torch.Tensor:
    """Jagged GDPA: for every sequence b and head h, ``O = (act(Q K^T) * qk_scale) V``.

    Same signature as the reference entry point.  ``query`` is ``[total_q, H, D]``, ``key`` and
    ``value`` are ``[total_kv, H_kv, D]`` with ``H`` a multiple of ``H_kv`` (grouped-query attention when
    smaller; bf16, D in {64, 128}); ``query_offset`` / ``key_offset`` are
    ``[B + 1]`` int32 or int64 prefix sums.  ``qk_scale=None`` means 1.0, as in the reference
    (:3148-3149).  ``activation`` is a reference activation name, or ``"softmax"`` (forward and
    backward), for which ``qk_scale`` multiplies the scores before the exponential.

    Scheduling knobs of the reference (``seq_index``, ``enable_persistent``, ``enable_tma``,
    ``enable_ws``, ``use_dq_atomic_add``, ``bwd_opt_tech``, ``allow_tf32``, ``total_num_objects``) are
    accepted and ignored: scheduling is internal.  ``ad_to_request_offset`` (one KV sequence index per Q
    sequence, so that many Q sequences share one KV sequence) is supported for the forward only;
    ``window_size=W`` keeps only pairs of sequence-local positions with ``|q - kv| <= W``;
    ``broadcast_q`` (one Q sequence shared by the whole batch) and ``ensemble_activation_list`` (one
    activation id per head) are composed on the host from calls of the same kernels;
    ``use_start_end_offsets`` (offsets ``[start_0, end_0, start_1, end_1, ...]``: sequences may share or overlap
    K / V rows; dK and dV are then summed in fp32 over the sequences that read a row) is supported forward and
    backward.  Every other
    non-default option raises, as the reference does for masks and causality (:3138-3139).
    """
    if attn_mask is not None:
        raise NotImplementedError("attn_mask/bias unsupported")
    if is_causal:
        raise NotImplementedError("Causal unsupported")
    unsupported = {
        "attn_offset": attn_offset,
        "ts_encoding_params": ts_encoding_params,
        "ts_event_request_even_params": ts_event_request_even_params,
        "ts_event_request_log_params": ts_event_request_log_params,
        "ts_adjacent_event_log_params": ts_adjacent_event_log_params,
        "ts_encoding_bucket_values": ts_encoding_bucket_values,
        "ts_event_request_even_bucket_values": ts_event_request_even_bucket_values,
        "ts_event_request_log_bucket_values": ts_event_request_log_bucket_values,
        "ts_adjacent_event_log_bucket_values": ts_adjacent_event_log_bucket_values,
        "pos_emb_params": pos_emb_params, "pos_emb_bucket_values": pos_emb_bucket_values,
    }
    for name, val in unsupported.items():
        if val is not None:
            raise NotImplementedError(f"{name} is not supported by this implementation")
    act_id = activation_string_to_int(activation)
    scale = 1.0 if qk_scale is None else float(qk_scale)
    if use_start_end_offsets:
        # reference: :3142-3146 (no packed layouts, no broadcast_q, total_num_objects required), output rows of
        # sequence b at query_offset[2 b] (:3156-3157, :625), output of total_num_objects rows (:3015-3024)
        if key is None or value is None or broadcast_q:
            raise ValueError("fused_qkv/fused_kv/broadcast_q not supported with start/end offsets")
        if total_num_objects is None:
            raise ValueError("total_num_objects must be provided")
        if int(total_num_objects) != query.shape[0]:
            raise NotImplementedError("total_num_objects must equal the number of query rows")
        if ad_to_request_offset is not None or ensemble_activation_list or output_offset is not None:
            raise NotImplementedError("start/end offsets together with ad_to_request_offset, ensemble_activation_list or "
                                      "output_offset are not supported")
        window = -1 if window_size is None else int(window_size)
        if window_size is not None and window < 0:
            raise ValueError("window_size must be non-negative")
        if act_id == SOFTMAX_ID:
            return torch.ops.gdpa.generalized_dot_product_attention_softmax(
                expect_contiguous(query), key, value, query_offset.contiguous(), key_offset.contiguous(), int(max_seq_len_q),
                int(max_seq_len_kv), scale, window, True)[0]
        return torch.ops.gdpa.generalized_dot_product_attention(
            expect_contiguous(query), key, value, query_offset.contiguous(), key_offset.contiguous(), int(max_seq_len_q),
            int(max_seq_len_kv), scale, act_id, window, True)
    if output_offset is not None and not broadcast_q:
        raise NotImplementedError("output_offset is supported together with broadcast_q only")
    # Packed layouts of the reference (:605-622): query = [T, H, 3D] with key = value = None, or
    # key = [T, H, 2D] with value = None.  The slices are strided views the kernels read in place.
    if key is None and value is None:
        if broadcast_q:  # the reference asserts the same (:3143-3145 for offsets, :606 for the layout)
            raise ValueError("broadcast_q cannot be combined with a fused QKV tensor")
        if query.shape[-1] % 3 != 0:
            raise ValueError("a fused QKV tensor must have a last dimension of 3 * head_dim")
        query, key, value = expect_contiguous(query).split(query.shape[-1] // 3, dim=-1)
    elif value is None:
        if key.shape[-1] % 2 != 0:
            raise ValueError("a fused KV tensor must have a last dimension of 2 * head_dim")
        query = expect_contiguous(query)
        key, value = expect_contiguous(key).split(key.shape[-1] // 2, dim=-1)
    elif key is None:
        raise ValueError("value given without key")
    else:
        query = expect_contiguous(query)
        key = expect_contiguous(key)
        value = expect_contiguous(value)
    window = -1 if window_size is None else int(window_size)
    if window_size is not None and window < 0:
        raise ValueError("window_size must be non-negative")
    if broadcast_q:
        if ad_to_request_offset is not None:
            raise NotImplementedError("broadcast_q together with ad_to_request_offset is not supported")
        query, query_offset = _broadcast_query(query, query_offset, key_offset, output_offset)
    if ensemble_activation_list:
        if ad_to_request_offset is not None:
            raise NotImplementedError("ensemble_activation_list together with ad_to_request_offset is not supported")
        return _ensemble(query, key, value, query_offset, key_offset, int(max_seq_len_q), int(max_seq_len_kv), scale,
                         act_id, window, [int(a) for a in ensemble_activation_list])
    if ad_to_request_offset is not None:
        return torch.ops.gdpa.generalized_dot_product_attention_shared_kv(
            query, key, value, query_offset, key_offset, ad_to_request_offset, int(max_seq_len_q), int(max_seq_len_kv),
            scale, act_id, window
        )
    return _dispatch(query, key, value, query_offset, key_offset, int(max_seq_len_q), int(max_seq_len_kv), scale, act_id,
                     window)


def _dispatch(query, key, value, query_offset, key_offset, max_q: int, max_kv: int, scale: float, act_id: int,
              window: int) -> torch.Tensor:
    if act_id == SOFTMAX_ID:
        # the trainable softmax variant keeps the log-sum-exp of the forward for its backward
        return torch.ops.gdpa.generalized_dot_product_attention_softmax(
            query, key, value, query_offset, key_offset, max_q, max_kv, scale, window
        )[0]
    return torch.ops.gdpa.generalized_dot_product_attention(
        query, key, value, query_offset, key_offset, max_q, max_kv, scale, act_id, window
    )


def _broadcast_query(query, query_offset, key_offset, output_offset):
    """``broadcast_q`` of the reference (:949-952, :3028, :3088-3089): ``query`` holds ONE sequence
    (``query_offset = [0, Lq]``) that every KV sequence of the batch attends with; the output is
    ``[B * Lq, H, D]`` with the rows of batch element z at ``output_offset[z]``, and dQ is the sum over the
    batch.  Composed on the host: the Q rows are repeated B times (a tensor of the size of the output) and
    the ordinary operator runs on them, so autograd sums dQ over the batch.  ``output_offset`` must be the
    dense layout ``[0, Lq, 2 Lq, ...]`` (the only one that fills the reference's output tensor); it is
    built here when it is not given."""
    if query_offset.numel() != 2:
        raise ValueError("broadcast_q expects a single query sequence: query_offset = [0, Lq]")
    batch = key_offset.numel() - 1
    lq = query.shape[0]
    if output_offset is None:
        output_offset = torch.arange(batch + 1, device=query.device, dtype=key_offset.dtype) * lq
    elif output_offset.numel() != batch + 1:
        raise ValueError("output_offset must have one entry per KV sequence plus one")
    elif _validate_offsets or not output_offset.is_cuda:
        # a device tensor is compared only when offset validation is on (the comparison synchronises)
        dense = torch.arange(batch + 1, dtype=torch.int64) * lq
        if not torch.equal(output_offset.detach().to("cpu", torch.int64), dense):
            raise ValueError("output_offset must be the dense layout [0, Lq, 2 Lq, ...]")
    return query.repeat(batch, 1, 1), output_offset.to(key_offset.dtype).contiguous()


def _ensemble(query, key, value, query_offset, key_offset, max_q, max_kv, scale, act_id, window,
              ensemble: List[int]) -> torch.Tensor:
    """Per-head activations (the reference's ``ensemble_activation_list``, :958-961: head i < len(list)
    uses activation id list[i], the other heads the base activation).  Composed on the host: heads are cut
    into runs of equal activation (aligned to K/V heads under grouped-query attention), each run is one
    call of the operator on strided head slices, and the outputs are concatenated along the head axis, so
    autograd assembles the gradients."""
    H, Hkv = query.shape[1], key.shape[1]
    if Hkv < 1 or H % Hkv != 0:
        raise ValueError("the number of query heads must be a multiple of the number of key/value heads")
    G = H // Hkv
    acts = [ensemble[h] if h < len(ensemble) else act_id for h in range(H)]
    for a in set(acts):
        if a != SOFTMAX_ID and a not in int_to_activation:
            raise ValueError(f"Unsupported activation id: {a}")
    # units of (first query head, last + 1, first K/V head, last + 1, activation): whole K/V heads whose
    # query heads agree, else single query heads; neighbouring whole-head units of one activation merge
    units = []
    for kvh in range(Hkv):
        lo, hi = kvh * G, (kvh + 1) * G
        if len(set(acts[lo:hi])) == 1:
            if units and units[-1][4] == acts[lo] and units[-1][1] == lo and units[-1][5]:
                units[-1] = (units[-1][0], hi, units[-1][2], kvh + 1, acts[lo], True)
            else:
                units.append((lo, hi, kvh, kvh + 1, acts[lo], True))
        else:
            units.extend((h, h + 1, kvh, kvh + 1, acts[h], False) for h in range(lo, hi))
    outs = [
        _dispatch(query[:, lo:hi], key[:, klo:khi], value[:, klo:khi], query_offset, key_offset, max_q, max_kv, scale,
                  act, window)
        for lo, hi, klo, khi, act, _ in units
    ]
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


def quantize_fp8_blockwise(x: torch.Tensor, offsets: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantise a jagged ``[total, H, D]`` tensor (bf16 or fp32, CUDA) to FP8 e4m3 with one fp32 scale per
    (sequence-local 128-token block, head): ``scale = max(amax / 448, 1e-12)`` over the block.

    Returns ``(x_fp8, scales[rows, H], block_offsets[B + 1])`` where block ``j`` of sequence ``b`` is row
    ``block_offsets[b] + j`` of ``scales`` (``rows = total // 128 + B`` is an upper bound of the number of blocks;
    rows past ``block_offsets[B]`` are zero).  Runs in the kernel library (``gdpa_quantize_fp8_blockwise``), without
    a host synchronisation; it is the producer of the inputs of :func:`generalized_dot_product_attention_fp8`.
    """
    if not x.is_cuda or x.dim() != 3 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("quantize_fp8_blockwise expects a CUDA [total, H, D] tensor of bf16 or fp32")
    if offsets.dtype not in (torch.int32, torch.int64) or offsets.device != x.device or offsets.dim() != 1:
        raise ValueError("offsets must be a 1-D int32 / int64 tensor on the device of x")
    x = x.contiguous()
    offsets = offsets.contiguous()
    total, H, D = x.shape
    batch = offsets.numel() - 1
    rows = total // 128 + batch
    with torch.cuda.device(x.device):
        x8 = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.zeros(max(rows, 1), H, dtype=torch.float32, device=x.device)
        blk_off = torch.empty(batch + 1, dtype=offsets.dtype, device=x.device)
        p = _cabi.GdpaQuantParams()
        p.struct_size = C.sizeof(_cabi.GdpaQuantParams)
        p.in_is_fp32 = int(x.dtype == torch.float32)
        p.x, p.x8, p.scales = x.data_ptr(), x8.data_ptr(), scales.data_ptr()
        p.offsets, p.block_offsets = offsets.data_ptr(), blk_off.data_ptr()
        p.offsets_are_int64 = int(offsets.dtype == torch.int64)
        p.batch, p.total, p.heads, p.head_dim, p.scale_rows = batch, total, H, D, max(rows, 1)
        _cabi.check(_cabi.lib.gdpa_quantize_fp8_blockwise(C.byref(p), _stream_ptr()), "gdpa_quantize_fp8_blockwise")
    return x8, scales, blk_off


def generalized_dot_product_attention_fp8(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    q_scales: torch.Tensor,
    k_scales: torch.Tensor,
    v_scales: torch.Tensor,
    q_block_offsets: torch.Tensor,
    kv_block_offsets: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    max_seq_len_q: int,
    max_seq_len_kv: int,
    qk_scale: Optional[float] = None,
    activation: str = "softmax",
) -> torch.Tensor:
    """Low-precision forward: FP8 e4m3 Q/K/V with per-128-token-block fp32 scales, bf16 output.
    Mirrors the reference's FP8 forward (gdpa/src/interface.py:1053 output dtype rule)."""
    act_id = activation_string_to_int(activation)
    scale = 1.0 if qk_scale is None else float(qk_scale)
    return torch.ops.gdpa.generalized_dot_product_attention_fp8(
        expect_contiguous(query), expect_contiguous(key), expect_contiguous(value), q_scales, k_scales, v_scales,
        q_block_offsets, kv_block_offsets, query_offset, key_offset, int(max_seq_len_q), int(max_seq_len_kv), scale,
        act_id,
    )


def _valid_pairs(query_offset: torch.Tensor, key_offset: torch.Tensor, max_q: int, max_kv: int) -> int:
    """sum over sequences of Lq * Lkv (lengths clamped like the kernels clamp them).  Reads the offsets
    on the host when they are real tensors; for meta / fake tensors falls back to batch * max_q * max_kv."""
    batch = query_offset.shape[0] - 1
    if query_offset.is_meta or key_offset.is_meta or type(query_offset).__name__ == "FakeTensor":
        return batch * int(max_q) * int(max_kv)
    qo = query_offset.detach().to("cpu", torch.int64)
    ko = key_offset.detach().to("cpu", torch.int64)
    lq = (qo[1:] - qo[:-1]).clamp(0, int(max_q))
    lk = (ko[1:] - ko[:-1]).clamp(0, int(max_kv))
    return int((lq * lk).sum())


def _register_flop_formulas() -> None:
    """Let torch.utils.flop_counter.FlopCounterMode see the operator, as the reference does
    (gdpa/triton/triton_generalized_dot_product_attention.py:4051, :4137): 4 H D sum(Lq Lkv) forward,
    2.5x that backward, valid jagged pairs only."""
    try:
        from torch.utils.flop_counter import register_flop_formula
    except ImportError:  # pragma: no cover
        return

    @register_flop_formula(torch.ops.gdpa.generalized_dot_product_attention, get_raw=True)
    def _fwd_flops(query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, *args, **kwargs) -> int:
        return 4 * query.shape[1] * query.shape[2] * _valid_pairs(query_offset, key_offset, max_seq_len_q, max_seq_len_kv)

    @register_flop_formula(torch.ops.gdpa.generalized_dot_product_attention_backward, get_raw=True)
    def _bwd_flops(do, query, key, value, query_offset, key_offset, max_seq_len_q, max_seq_len_kv, *args, **kwargs) -> int:
        return 10 * query.shape[1] * query.shape[2] * _valid_pairs(query_offset, key_offset, max_seq_len_q, max_seq_len_kv)


_register_flop_formulas()
