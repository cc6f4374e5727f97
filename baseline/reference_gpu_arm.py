#!/usr/bin/env python
"""Same-box comparator: the reference's own Blackwell GDPA kernels (CuteDSL, `flash_attn_varlen_func`,
gdpa/src/interface.py:2223 of the reference) timed on the cells of the reference's published workload
(gdpa/scripts/benchmark.py:176-185, :574-598), the way that script times them (`run_fwd` :239-265, `run_bwd`
:330-385: tile maps precomputed outside the timed call, backward through autograd with retain_graph).

    baseline/install_reference.sh /path/to/ads_model_kernel_library      # once, where the reference is mounted
    python baseline/reference_gpu_arm.py [--small-only] [--sets self_s1,...] [--lengths 256,...]
    python baseline/reference_gpu_arm.py --accuracy      # forward error of both implementations, one small batch

The reference's kernels are Python DSL sources that compile at their first call, against the nvidia-cutlass-dsl
package of the machine (the reference pins another version), and their waits have no time limit.  So every cell
runs in a child process with a time limit; the first cell is a small one (B=8, L=512); the first failure or
time-out ends the run and is reported as one JSON line with `"unavailable"`.  One JSON line per cell otherwise.
This arm is a reported comparison; nothing in the package or in the tests depends on it.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def worker(kind: str, lengths, B: int, mode: str, cell_ms: float) -> None:
    """All lengths of one (set, pass) in one process, so that the kernels compile once."""
    import numpy as np
    import torch

    sys.path.insert(0, REF)
    from ads_mkl.ops.oss.gdpa.src.interface import flash_attn_varlen_func, precompute_for_varline_load_balancing

    torch.manual_seed(2025)
    H, D = 4, 128
    dev = torch.device("cuda", 0)
    grad = mode == "bwd"
    for L in lengths:
        rng = np.random.default_rng(2025 + L)
        lq = rng.integers(1, L + 1, B) if kind == "self_s05" else np.full(B, L)
        dff = 256 if kind == "cross_kv256" else L
        q_off = torch.from_numpy(np.concatenate([[0], np.cumsum(lq)])).to(torch.int32).to(dev)
        kv_off = (torch.arange(B + 1, dtype=torch.int32) * dff).to(dev)
        q = torch.randn(int(lq.sum()), H, D, dtype=torch.bfloat16, device=dev, requires_grad=grad)
        k = torch.randn(B * dff, H, D, dtype=torch.bfloat16, device=dev, requires_grad=grad)
        v = torch.randn(B * dff, H, D, dtype=torch.bfloat16, device=dev, requires_grad=grad)
        tq = precompute_for_varline_load_balancing(q, q_off, kv_off)
        kw = dict(q=q, k=k, v=v, cu_seqlens_q=q_off, cu_seqlens_k=kv_off, max_seqlen_q=int(lq.max()), max_seqlen_k=dff,
                  prefer_persistent=True, tile_to_batch_q=tq[0], tile_to_head_q=tq[1], tile_to_block_q=tq[2], activation="fast_gelu")
        if grad:
            tk = precompute_for_varline_load_balancing(q, q_off, kv_off, is_bwd=True)
            kw.update(tile_to_batch_k=tk[0], tile_to_head_k=tk[1], tile_to_block_k=tk[2])
        pairs = float((lq.astype(np.float64) * dff).sum())
        flops = 4.0 * H * D * pairs * (2.5 if grad else 1.0)
        if grad:
            res = flash_attn_varlen_func(**kw)
            out = res[0] if isinstance(res, (tuple, list)) else res
            dout = torch.randn_like(out)

            def fn():
                q.grad = k.grad = v.grad = None
                out.backward(dout, retain_graph=True)
        else:
            def fn():
                with torch.no_grad():
                    flash_attn_varlen_func(**kw)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); torch.cuda.synchronize()
        reps = int(min(200, max(5, cell_ms / max(a.elapsed_time(b), 1e-3))))
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for x, y in evs:
            x.record(); fn(); y.record()
        torch.cuda.synchronize()
        ms = float(np.median([x.elapsed_time(y) for x, y in evs]))
        print("RESULT " + json.dumps({"impl": "reference_kernel", "metric": f"gdpa_{mode}_useful_tflops",
                                      "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": reps,
                                      "config": {"workload": f"ref_{kind}_{mode}_L{L}", "batch": B, "heads": H, "head_dim": D,
                                                 "activation": "fast_gelu", "api": "flash_attn_varlen_func (CuteDSL, persistent)"}}),
              flush=True)
        del q, k, v
        torch.cuda.empty_cache()


def accuracy_worker() -> None:
    """Forward of both implementations on one small batch (B=8, L=512, H=4, D=128, fast_gelu, scale 1) at three input
    magnitudes, against the same product evaluated in fp32 by torch (tanh form of GELU, gdpa/triton/math.py:150-165
    of the reference; P not rounded).  One RESULT line per (implementation, magnitude)."""
    import torch

    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.dirname(HERE))
    from ads_mkl.ops.oss.gdpa.src.interface import flash_attn_varlen_func
    import ads_model_kernel_library_b200.gdpa  # noqa: F401  (registers torch.ops.gdpa)
    from ads_model_kernel_library_b200.gdpa.math import activation_string_to_int

    B, L, H, D = 8, 512, 4, 128
    dev = torch.device("cuda", 0)
    off = (torch.arange(B + 1, dtype=torch.int32) * L).to(dev)
    act_id = activation_string_to_int("fast_gelu")
    for std in (0.2, 0.35, 0.5):
        g = torch.Generator(device=dev).manual_seed(7)
        q, k, v = ((torch.randn(B * L, H, D, generator=g, device=dev) * std).to(torch.bfloat16) for _ in range(3))
        qf, kf, vf = (t.float().view(B, L, H, D).permute(0, 2, 1, 3) for t in (q, k, v))
        s = qf @ kf.transpose(-1, -2)
        exact = (torch.nn.functional.gelu(s, approximate="tanh") @ vf).permute(0, 2, 1, 3).reshape(B * L, H, D)
        res = flash_attn_varlen_func(q=q, k=k, v=v, cu_seqlens_q=off, cu_seqlens_k=off, max_seqlen_q=L, max_seqlen_k=L,
                                     softmax_scale=1.0, activation="fast_gelu")
        outs = {"reference_kernel": (res[0] if isinstance(res, (tuple, list)) else res).float(),
                "this_library": torch.ops.gdpa.generalized_dot_product_attention(q, k, v, off, off, L, L, 1.0, act_id).float()}
        rms = exact.pow(2).mean().sqrt().item()
        for impl, o in outs.items():
            err = o - exact
            print("RESULT " + json.dumps({"impl": impl, "check": "forward against fp32 torch, fast_gelu, scale 1", "input_std": std,
                                          "score_std": s.std().item(), "share_of_scores_beyond_2": (s.abs() > 2).float().mean().item(),
                                          "out_rms": rms, "rel_rms_err": err.pow(2).mean().sqrt().item() / rms,
                                          "max_abs_err": err.abs().max().item()}), flush=True)


def run_cells(kind, lengths, B, mode, cell_ms, limit_s):
    """Results of the cells that finished, and an error text if the child failed or ran out of time."""
    cmd = [sys.executable, os.path.abspath(__file__), "--worker", kind, ",".join(str(x) for x in lengths), str(B), mode, str(cell_ms)]
    err = None
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=limit_s)
        out, code, tail = r.stdout, r.returncode, r.stderr
    except subprocess.TimeoutExpired as e:
        out = e.stdout.decode() if isinstance(e.stdout, bytes) else (e.stdout or "")
        code, tail = None, ""
        err = f"no result within {limit_s} s (compile or kernel did not finish)"
    results = [json.loads(line[7:]) for line in out.splitlines() if line.startswith("RESULT ")]
    if err is None and len(results) < len(lengths):
        last = (tail.strip().splitlines() or out.strip().splitlines() or ["no output"])[-1]
        err = f"exit code {code}: {last[:400]}"
    return results, err


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", nargs=5, default=None)
    ap.add_argument("--small-only", action="store_true")
    ap.add_argument("--accuracy", action="store_true",
                    help="instead of timing: forward error of the reference's kernel and of this library on one small batch")
    ap.add_argument("--sets", default="self_s1,self_s05,cross_kv256")
    ap.add_argument("--lengths", default="256,512,1024,2048")
    ap.add_argument("--cell-ms", type=float, default=600.0)
    ap.add_argument("--limit-s", type=float, default=420.0)
    args = ap.parse_args()
    if args.worker:
        kind, lengths, B, mode, cell_ms = args.worker
        if kind == "accuracy":
            accuracy_worker()
        else:
            worker(kind, [int(x) for x in lengths.split(",")], int(B), mode, float(cell_ms))
        return
    if not os.path.isdir(os.path.join(REF, "ads_mkl", "ops", "oss", "gdpa")):
        print(json.dumps({"impl": "reference_kernel", "unavailable": "baseline/_ref is empty: run baseline/install_reference.sh first"}))
        return
    if args.accuracy:
        results, err = run_cells("accuracy", [0] * 6, 8, "fwd", 0.0, args.limit_s)
        for res in results:
            print(json.dumps(res), flush=True)
        if err is not None:
            print(json.dumps({"impl": "reference_kernel", "unavailable": f"accuracy check: {err}"}), flush=True)
        return
    groups = [("self_s1", [512], 8, "fwd"), ("self_s1", [512], 8, "bwd")]  # a small case first
    if not args.small_only:
        lengths = [int(x) for x in args.lengths.split(",")]
        groups += [(k, lengths, 1152, mode) for k in args.sets.split(",") for mode in ("fwd", "bwd")]
    for kind, lengths, B, mode in groups:
        results, err = run_cells(kind, lengths, B, mode, args.cell_ms, args.limit_s)
        for res in results:
            print(json.dumps(res), flush=True)
        if err is not None:
            print(json.dumps({"impl": "reference_kernel", "unavailable": f"ref_{kind}_{mode} (B={B}, L={lengths}): {err}"}), flush=True)
            return


if __name__ == "__main__":
    main()
