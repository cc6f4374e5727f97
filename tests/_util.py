"""Helpers shared by the GPU parity tests: seeded jagged inputs and comparison with the oracle."""
from __future__ import annotations

import numpy as np
import torch

from oracle import gdpa_oracle as orc

# Tolerance of the bf16 kernels against the fp32 oracle evaluated on the bf16-rounded inputs.
ATOL = 2e-2
RTOL = 2e-2


def jagged_inputs(q_lens, kv_lens, heads, head_dim, seed=0, std=1.0, device="cuda", offset_dtype=torch.int64,
                  dtype=torch.bfloat16):
    q_lens = np.asarray(q_lens, dtype=np.int64)
    kv_lens = np.asarray(kv_lens, dtype=np.int64)
    qo = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=offset_dtype)
    ko = torch.tensor(np.concatenate([[0], np.cumsum(kv_lens)]), dtype=offset_dtype)
    g = torch.Generator().manual_seed(seed)
    tq, tk = int(qo[-1]), int(ko[-1])
    q = (torch.randn(tq, heads, head_dim, generator=g) * std).to(dtype)
    k = (torch.randn(tk, heads, head_dim, generator=g) * std).to(dtype)
    v = (torch.randn(tk, heads, head_dim, generator=g) * std).to(dtype)
    do = (torch.randn(tq, heads, head_dim, generator=g) * std).to(dtype)
    cpu = dict(q=q, k=k, v=v, do=do, qo=qo, ko=ko)
    dev = {n: t.to(device) for n, t in cpu.items()}
    return cpu, dev


def oracle_forward(cpu, activation, scale):
    return orc.gdpa_forward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"], activation, scale)


def oracle_forward_backward(cpu, activation, scale):
    return orc.gdpa_forward_backward(cpu["q"].float(), cpu["k"].float(), cpu["v"].float(), cpu["qo"], cpu["ko"],
                                     cpu["do"].float(), activation, scale)


def assert_close(actual: torch.Tensor, expected: torch.Tensor, what: str, atol=ATOL, rtol=RTOL):
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    err = (a - e).abs()
    bad = err > (atol + rtol * e.abs())
    assert not bad.any(), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements outside atol={atol} rtol={rtol}; "
        f"max abs err {float(err.max()):.4g}, max abs ref {float(e.abs().max()):.4g}"
    )
