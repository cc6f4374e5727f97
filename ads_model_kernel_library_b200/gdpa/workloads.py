"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark
configurations (stand-ins for the reference's own generator, gdpa/utils/utils.py:66-136; no public
dataset is involved).  Lengths come from ``numpy.random.default_rng(seed)``, values from a
``torch.Generator`` on the requested device."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch


@dataclass
class Workload:
    name: str
    q_lens: np.ndarray
    kv_lens: np.ndarray
    heads: int
    head_dim: int
    activation: str
    qk_scale: float
    std: float
    mode: str  # "fwd" or "fwd_bwd"
    shared_offsets: bool

    @property
    def max_q(self) -> int:
        return int(self.q_lens.max()) if self.q_lens.size else 0

    @property
    def max_kv(self) -> int:
        return int(self.kv_lens.max()) if self.kv_lens.size else 0


def _lognormal(rng, median, sigma, lo, hi, n):
    return np.clip(np.rint(np.exp(rng.normal(np.log(median), sigma, n))), lo, hi).astype(np.int64)


def make_workload(name: str, batch: Optional[int] = None) -> Workload:
    """Lengths and parameters of a named configuration; ``batch`` overrides the number of
    sequences (same distribution, same seed) for reduced-size runs."""
    if name == "c1_cpu_small":
        rng = np.random.default_rng(0)
        b = batch or 8
        lq, lk = rng.integers(16, 257, b), rng.integers(16, 257, b)
        return Workload(name, lq, lk, 2, 64, "gelu_approx", 1.0 / int(lk.max()), 1.0, "fwd_bwd", False)
    if name == "c2_fwd_silu_lognormal":
        rng = np.random.default_rng(1)
        b = batch or 1024
        lq = _lognormal(rng, 256, 0.75, 16, 2048, b)
        lk = _lognormal(rng, 1024, 0.75, 16, 4096, b)
        return Workload(name, lq, lk, 4, 128, "silu", 1.0 / int(lk.max()), 1.0, "fwd", False)
    if name == "c3_fwd_bwd_gelu_uniform":
        rng = np.random.default_rng(2)
        b = batch or 512
        ln = rng.integers(512, 4097, b)
        return Workload(name, ln, ln.copy(), 8, 128, "gelu_approx", 1.0 / int(ln.max()), 0.5, "fwd_bwd", True)
    if name == "c4_fp8_softmax":
        rng = np.random.default_rng(3)
        b = batch or 1024
        ln = rng.integers(128, 2049, b)
        return Workload(name, ln, ln.copy(), 4, 128, "softmax", 1.0 / float(np.sqrt(128.0)), 1.0, "fwd", True)
    if name == "c5_zipf_sharded":
        rng = np.random.default_rng(5)
        b = batch or 8192
        ln = 32 * np.minimum(rng.zipf(1.2, b), 256).astype(np.int64)
        return Workload(name, ln, ln.copy(), 4, 128, "gelu_approx", 1.0 / int(ln.max()), 0.5, "fwd_bwd", True)
    raise KeyError(name)


WORKLOADS = ("c1_cpu_small", "c2_fwd_silu_lognormal", "c3_fwd_bwd_gelu_uniform", "c4_fp8_softmax", "c5_zipf_sharded")


def useful_flops(q_lens, kv_lens, heads: int, head_dim: int, mode: str = "fwd") -> int:
    """4 H D sum(Lq Lkv) forward, x2.5 backward, x3.5 both; valid jagged pairs only
    (same accounting as gdpa/scripts/benchmark.py:212-222, :668-674)."""
    pairs = int(np.sum(np.asarray(q_lens, dtype=np.int64) * np.asarray(kv_lens, dtype=np.int64)))
    fwd = 4 * heads * head_dim * pairs
    return {"fwd": fwd, "bwd": fwd * 5 // 2, "fwd_bwd": fwd * 7 // 2}[mode]


def make_tensors(w: Workload, device, seed: int = 0, dtype=torch.bfloat16, with_grad_out: bool = False,
                 seq_range=None) -> Dict[str, torch.Tensor]:
    """Random Q, K, V (and dO) of a workload, or of the sequence range ``seq_range=(start, end)`` of
    it, generated on ``device``; offsets are int64 exclusive prefix sums."""
    lq, lk = w.q_lens, w.kv_lens
    if seq_range is not None:
        lq, lk = lq[seq_range[0]:seq_range[1]], lk[seq_range[0]:seq_range[1]]
    qo = np.concatenate([[0], np.cumsum(lq)]).astype(np.int64)
    ko = np.concatenate([[0], np.cumsum(lk)]).astype(np.int64)
    g = torch.Generator(device=device).manual_seed(seed)
    shape_q = (int(qo[-1]), w.heads, w.head_dim)
    shape_k = (int(ko[-1]), w.heads, w.head_dim)

    def rnd(shape):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * w.std).to(dtype)

    out = {
        "q": rnd(shape_q), "k": rnd(shape_k), "v": rnd(shape_k),
        "q_offsets": torch.from_numpy(qo).to(device), "kv_offsets": torch.from_numpy(ko).to(device),
    }
    if with_grad_out:
        out["do"] = rnd(shape_q)
    return out
