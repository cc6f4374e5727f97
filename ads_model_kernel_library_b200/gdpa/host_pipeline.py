"""Host-buffer entry point: GDPA forward + backward over a jagged batch that lives in (pinned) host
memory, with the host<->device copies overlapped with the kernels.

The batch is cut into token-balanced ranges of sequences (the same planner that shards a batch over
GPUs); range i+1 is copied to the device while range i is computed and range i-1 is copied back, on
three CUDA streams.  Sequences are independent, so the result is identical to one call on the whole
batch.  This is plumbing around the operator, for callers whose data arrives from the host every
step; callers whose tensors already live on the device call the operator directly.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from .math import activation_string_to_int
from .sharding import plan_token_balanced_shards


def forward_backward_host(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    grad_out: torch.Tensor,
    query_offset: torch.Tensor,
    key_offset: torch.Tensor,
    qk_scale: Optional[float] = None,
    activation: str = "raw",
    out: Optional[Dict[str, torch.Tensor]] = None,
    n_chunks: int = 32,
    device=None,
) -> Dict[str, torch.Tensor]:
    """O, dQ, dK, dV (host tensors, pinned when allocated here) of jagged GDPA for host inputs.

    ``query`` / ``grad_out`` are ``[Tq, H, D]``, ``key`` / ``value`` ``[Tk, H, D]`` bf16 CPU tensors
    (pinned memory makes the copies asynchronous), offsets are CPU integer tensors.  ``out`` may hold
    preallocated ``"o", "dq", "dk", "dv"`` host tensors to write into.  The function returns when the last
    device-to-host copy has finished: the host may read the results straight away.

    The returned dictionary also carries ``"timing"``: milliseconds of the host-to-device copies, the kernels and
    the device-to-host copies as measured by CUDA events on their three streams (they overlap, so they do not add
    up to the wall time), and the bytes copied each way.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    act_id = activation_string_to_int(activation)
    scale = 1.0 if qk_scale is None else float(qk_scale)
    qo = query_offset.detach().cpu().numpy().astype(np.int64)
    ko = key_offset.detach().cpu().numpy().astype(np.int64)
    lq, lk = np.diff(qo), np.diff(ko)
    n_chunks = max(1, min(int(n_chunks), len(lq)))
    ranges = [(s, e) for s, e in plan_token_balanced_shards(lq, lk, n_chunks) if e > s]
    if out is None:
        pin = query.is_pinned()
        out = {
            "o": torch.empty(query.shape, dtype=query.dtype, pin_memory=pin),
            "dq": torch.empty(query.shape, dtype=query.dtype, pin_memory=pin),
            "dk": torch.empty(key.shape, dtype=key.dtype, pin_memory=pin),
            "dv": torch.empty(value.shape, dtype=value.dtype, pin_memory=pin),
        }
    with torch.cuda.device(device):
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        marks = {name: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for name in ("h2d", "compute", "d2h")}
        marks["h2d"][0].record(s_in)
        marks["compute"][0].record(main)
        marks["d2h"][0].record(s_out)
        done = []
        h2d_bytes = d2h_bytes = 0
        for s, e in ranges:
            q0, q1, k0, k1 = int(qo[s]), int(qo[e]), int(ko[s]), int(ko[e])
            off_q = torch.from_numpy(qo[s:e + 1] - q0)
            off_k = torch.from_numpy(ko[s:e + 1] - k0)
            with torch.cuda.stream(s_in):
                dq_, dk_, dv_, do_ = (t.to(device, non_blocking=True) for t in
                                      (query[q0:q1], key[k0:k1], value[k0:k1], grad_out[q0:q1]))
                oq_, ok_ = off_q.to(device, non_blocking=True), off_k.to(device, non_blocking=True)
                h2d_bytes += sum(t.numel() * t.element_size() for t in (dq_, dk_, dv_, do_))
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            main.wait_event(ev_in)
            for t in (dq_, dk_, dv_, do_, oq_, ok_):
                t.record_stream(main)
            max_q, max_k = int(lq[s:e].max()), int(lk[s:e].max())
            o = torch.ops.gdpa.generalized_dot_product_attention(dq_, dk_, dv_, oq_, ok_, max_q, max_k, scale, act_id)
            gq, gk, gv = torch.ops.gdpa.generalized_dot_product_attention_backward(
                do_, dq_, dk_, dv_, oq_, ok_, max_q, max_k, scale, act_id)
            ev_out = torch.cuda.Event()
            ev_out.record(main)
            s_out.wait_event(ev_out)
            with torch.cuda.stream(s_out):
                for t in (o, gq, gk, gv):
                    t.record_stream(s_out)
                out["o"][q0:q1].copy_(o, non_blocking=True)
                out["dq"][q0:q1].copy_(gq, non_blocking=True)
                out["dk"][k0:k1].copy_(gk, non_blocking=True)
                out["dv"][k0:k1].copy_(gv, non_blocking=True)
            d2h_bytes += sum(t.numel() * t.element_size() for t in (o, gq, gk, gv))
            done.append((o, gq, gk, gv))
        marks["h2d"][1].record(s_in)
        marks["compute"][1].record(main)
        marks["d2h"][1].record(s_out)
        main.wait_stream(s_out)
        # the copies into the host tensors are asynchronous: wait for the last one before handing the tensors back
        marks["d2h"][1].synchronize()
        out["timing"] = {name: a.elapsed_time(b) for name, (a, b) in marks.items()}
        out["timing"].update(h2d_bytes=h2d_bytes, d2h_bytes=d2h_bytes)
    return out
