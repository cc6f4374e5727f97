#!/usr/bin/env python
"""Benchmark of the GDPA hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one forward + backward pass of the operator over one jagged batch of synthetic input
(seeded; shapes and value distributions of the named workload).  The default workload is the
fwd+bwd BF16 configuration: B=512 sequences, H=8, D=128, Q=KV lengths uniform in [512, 4096],
GELU-tanh, scale 1/max_len, values N(0, 0.5).  With N > 1 (launched by torch.distributed.run, one
process per GPU) every rank runs its own batch of that configuration (weak scaling; sequences are
independent, so there is no collective on the data path) and the time is the maximum over ranks.
`--workload c5_zipf_sharded` instead splits the B=8192 Zipf batch by token-balanced offsets over
the ranks (strong scaling; on fewer than 8 GPUs each rank runs its range as several pieces, one
after another, so that the outputs and the fp32 dQ accumulator of one piece at a time fit in HBM).

Rank 0 prints ONE JSON line.  `value` is whole-job useful TFLOP/s (14 H D sum(Lq Lkv) per step,
valid jagged pairs only) with the inputs resident in HBM; `e2e` is the same metric through the
public Python entry point with pinned HOST buffers, host<->device copies inside the timed region.
`--impl reference` times the reference's eager PyTorch formulation (the CPU oracle port) on the
host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes per Q token of one launch (dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of
# 48 sequences of the default workload, H=8, D=128; see profiles/gdpa_*_kernel_bf16_d128_gelu_small_case.md).
# Traffic grows in proportion to the tokens, so a full launch is this figure times its Q tokens.
NCU_DRAM_BYTES_PER_TOKEN = {"gdpa_bwd_kernel": 2.347e9 / 114351, "gdpa_fwd_kernel": 0.928e9 / 114351}

METRIC = "gdpa_fwd_bwd_useful_tflops"
UNIT = "TFLOP/s"
DEFAULT_WORKLOAD = "c3_fwd_bwd_gelu_uniform"


def _peaks():
    """Measured denominators (driver-written file), else the pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "power_w_max": float(max(pw)),
                "samples": len(sm), "reasons": sorted(reasons)}


def _cpu_oracle_rate(workload_name: str, target_flops: float = 8e12):
    """Useful TFLOP/s of the eager fp32 formulation on the host cores, on the first sequences of the
    workload up to about `target_flops` of work."""
    from oracle import gdpa_oracle as orc
    from ads_model_kernel_library_b200.gdpa.workloads import make_workload, useful_flops

    w = make_workload(workload_name)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n, acc = 0, 0.0
    while n < len(w.q_lens) and (n == 0 or acc < target_flops):
        acc += 14.0 * w.heads * w.head_dim * float(w.q_lens[n]) * float(w.kv_lens[n])
        n += 1
    lq, lk = w.q_lens[:n], w.kv_lens[:n]
    qo = torch.from_numpy(np.concatenate([[0], np.cumsum(lq)]))
    ko = torch.from_numpy(np.concatenate([[0], np.cumsum(lk)]))
    g = torch.Generator().manual_seed(0)
    q = torch.randn(int(qo[-1]), w.heads, w.head_dim, generator=g) * w.std
    k = torch.randn(int(ko[-1]), w.heads, w.head_dim, generator=g) * w.std
    v = torch.randn(int(ko[-1]), w.heads, w.head_dim, generator=g) * w.std
    do = torch.randn(int(qo[-1]), w.heads, w.head_dim, generator=g) * w.std
    t0 = time.perf_counter()
    orc.gdpa_forward_backward(q, k, v, qo, ko, do, w.activation, w.qk_scale)
    dt = time.perf_counter() - t0
    fl = useful_flops(lq, lk, w.heads, w.head_dim, "fwd_bwd")
    return fl / dt / 1e12, dt, cores, f"first {n} sequences of {workload_name} ({int(qo[-1])} Q tokens), fwd+bwd fp32 eager, {dt:.1f} s"


def run_reference(args, rank: int):
    """The reference arm: the reference's own CPU formulation of the path (eager PyTorch fp32 per
    sequence, autograd backward) on all host cores, same metric and config."""
    if rank != 0:
        return
    from ads_model_kernel_library_b200.gdpa.workloads import make_workload

    w = make_workload(args.workload)
    vals, dts = [], []
    sample = ""
    for i in range(args.warmup + args.steps):
        v, dt, cores, sample = _cpu_oracle_rate(args.workload, target_flops=args.ref_flops)
        if i >= args.warmup:
            vals.append(v); dts.append(dt)
    value = float(np.mean(vals))
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(dts) * 1e3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": int(len(w.q_lens)), "heads": w.heads, "head_dim": w.head_dim,
                   "activation": w.activation, "pass": "fwd+bwd", "sampled": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the number of sequences (reduced-size runs)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--e2e-chunks", type=int, default=32)
    ap.add_argument("--activation", default=None, help="override the workload's activation (experiments)")
    ap.add_argument("--norms", action="store_true",
                    help="time the forward of the GDPA-plus-norm pipeline (layer norm of Q, Q residual, RMS norm) "
                         "instead of the workload's own pass, and the two row-norm kernels against the HBM roofline")
    ap.add_argument("--mxfp8", action="store_true",
                    help="with --workload c4_fp8_softmax: feed the forward MXFP8 inputs (e4m3 + e8m0 scale per 32 elements); "
                         "the three de-quantising passes are inside the timed step")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-flops", type=float, default=None, help="useful FLOPs of the CPU sample per step of the reference arm")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.ref_flops is None:  # keep the whole reference run within a few minutes
            args.ref_flops = 3e12 / max(1, args.steps + args.warmup)
        run_reference(args, rank)
        return

    if args.warmup < 3:
        args.warmup = 3
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import ads_model_kernel_library_b200.gdpa as G
    from ads_model_kernel_library_b200.gdpa import _cabi
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload, useful_flops

    w = make_workload(args.workload, batch=args.batch)
    if args.activation:
        w.activation = args.activation
    strong = args.workload == "c5_zipf_sharded"
    fp8 = args.workload == "c4_fp8_softmax" and not args.mxfp8
    mx = args.workload == "c4_fp8_softmax" and args.mxfp8
    assert not args.mxfp8 or mx, "--mxfp8 goes with --workload c4_fp8_softmax"
    if args.norms:
        assert not fp8 and w.activation != "softmax", "--norms needs a bf16 workload with an element-wise activation"
        w.mode = "fwd"
    fwd_only = w.mode == "fwd"
    metric = METRIC if not fwd_only else ("gdpa_fwd_norms_useful_tflops" if args.norms else "gdpa_fwd_useful_tflops")
    if strong:
        # token-balanced contiguous ranges; a rank's range is streamed in pieces that fit in HBM
        pieces_per_rank = max(1, 8 // world)
        shards = G.plan_token_balanced_shards(w.q_lens, w.kv_lens, world * pieces_per_rank)
        my_ranges = shards[rank * pieces_per_rank:(rank + 1) * pieces_per_rank]
    else:
        my_ranges = [(0, len(w.q_lens))]
    batches = []
    for i, (s, e) in enumerate(my_ranges):
        if e <= s:
            continue
        t = make_tensors(w, dev, seed=1000 * rank + i, with_grad_out=True, seq_range=(s, e))
        t["lq"], t["lk"] = w.q_lens[s:e], w.kv_lens[s:e]
        t["max_q"], t["max_kv"] = int(t["lq"].max()), int(t["lk"].max())
        if fp8:
            # quantise once, outside the timed region: FP8 tensors + per-block scales are the op's inputs
            t["q8"], t["sq"], t["qb"] = G.quantize_fp8_blockwise(t["q"].float(), t["q_offsets"])
            t["k8"], t["sk"], t["kb"] = G.quantize_fp8_blockwise(t["k"].float(), t["kv_offsets"])
            t["v8"], t["sv"], t["vb"] = G.quantize_fp8_blockwise(t["v"].float(), t["kv_offsets"])
        if mx:
            t["q8"], t["sfq"], _ = G.quantize_varlen_mxfp8_sf_only(t["q"], t["q_offsets"], 0)
            t["k8"], t["sfk"], _ = G.quantize_varlen_mxfp8_sf_only(t["k"], t["kv_offsets"], 0)
            t["v8"], t["sfv"], _ = G.quantize_varlen_mxfp8_sf_only(t["v"], t["kv_offsets"], 1)
        batches.append(t)
    flops_rank = sum(useful_flops(b["lq"], b["lk"], w.heads, w.head_dim, w.mode) for b in batches)
    tokens_rank = sum(int(b["lq"].sum() + b["lk"].sum()) for b in batches)

    def step():
        for b in batches:
            if fwd_only:
                with torch.no_grad():
                    if args.norms:
                        G.gdpa_megakernel(b["q"], b["k"], b["v"], b["q_offsets"], b["kv_offsets"], b["max_q"], b["max_kv"],
                                          qk_scale=w.qk_scale, activation=w.activation, fused_layernorm=True,
                                          fused_q_residual_add=True, fused_rms_norm=True)
                    elif mx:
                        G.generalized_dot_product_attention_mxfp8(b["q8"], b["k8"], b["v8"], b["sfq"], b["sfk"], b["sfv"],
                                                                  b["q_offsets"], b["kv_offsets"], b["max_q"], b["max_kv"],
                                                                  qk_scale=w.qk_scale, activation=w.activation)
                    elif fp8:
                        G.generalized_dot_product_attention_fp8(b["q8"], b["k8"], b["v8"], b["sq"], b["sk"], b["sv"], b["qb"],
                                                                b["kb"], b["q_offsets"], b["kv_offsets"], b["max_q"],
                                                                b["max_kv"], qk_scale=w.qk_scale, activation=w.activation)
                    else:
                        G.generalized_dot_product_attention(b["q"], b["k"], b["v"], b["q_offsets"], b["kv_offsets"],
                                                            b["max_q"], b["max_kv"], qk_scale=w.qk_scale,
                                                            activation=w.activation)
                continue
            q = b["q"].requires_grad_(True)
            k = b["k"].requires_grad_(True)
            v = b["v"].requires_grad_(True)
            o = G.generalized_dot_product_attention(q, k, v, b["q_offsets"], b["kv_offsets"], b["max_q"], b["max_kv"],
                                                    qk_scale=w.qk_scale, activation=w.activation)
            o.backward(b["do"])
            q.grad = k.grad = v.grad = None
            del o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert G.kernel_status() == 0, "a kernel wait ran out during warm-up"

    # ---- timed region: K steps, CUDA events on the launching stream, max over ranks ----------
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    bwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    launches0 = _cabi.lib.gdpa_launch_count()
    if rank == 0:
        sampler.start()
    barrier()
    e0.record()
    for i in range(args.steps):
        with G.kernel_timing(fwd=fwd_ev[i], bwd=bwd_ev[i]):
            step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = _cabi.lib.gdpa_launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(flops_rank), float(tokens_rank)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_step = float(t.item()) / args.steps
    total_flops, total_tokens = float(tot[0].item()), float(tot[1].item())
    value = total_flops / (ms_step * 1e-3) / 1e12
    assert G.kernel_status() == 0, "a kernel wait ran out during the timed region"

    # dominant kernel: the backward kernel (last call of each step carries the events)
    fwd_ms = float(np.mean([a.elapsed_time(b) for a, b in fwd_ev]))
    last = batches[-1]
    fwd_flops = useful_flops(last["lq"], last["lk"], w.heads, w.head_dim, "fwd")
    peaks = _peaks()
    peak = peaks["bf16_tflops_sustained"]
    fwd_part = {"kernel": "gdpa_fwd_kernel", "achieved": fwd_flops / (fwd_ms * 1e-3) / 1e12,
                "frac": fwd_flops / (fwd_ms * 1e-3) / 1e12 / peak, "kernel_ms": fwd_ms}
    if fwd_only:
        peak_note = peaks["source"] + " bf16_tflops_sustained"
        if fp8:
            peak_note += " (no measured FP8 rate on this pool: the bf16 rate is the denominator, nominal FP8 is 2x bf16)"
        roofline = {"bound": "tensor", "kernel": "gdpa_fwd_kernel", "achieved": fwd_part["achieved"], "peak": peak,
                    "unit": "TFLOP/s", "frac": fwd_part["frac"], "peak_source": peak_note, "traffic": None,
                    "kernel_ms": fwd_ms, "frac_of_nominal": fwd_part["achieved"] / (4500.0 if fp8 else 2250.0)}
    else:
        bwd_ms = float(np.mean([a.elapsed_time(b) for a, b in bwd_ev]))
        bwd_flops = useful_flops(last["lq"], last["lk"], w.heads, w.head_dim, "bwd")
        achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "gdpa_bwd_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak,
                    "peak_source": peaks["source"] + " bf16_tflops_sustained (kernel timed inside a long step)",
                    "traffic": (NCU_DRAM_BYTES_PER_TOKEN["gdpa_bwd_kernel"] * float(last["lq"].sum())
                                if (w.heads, w.head_dim) == (8, 128) else None),
                    "traffic_note": "bytes per launch, scaled by tokens from an ncu capture of 48 sequences",
                    "algorithmic_bytes": 16.0 * w.heads * w.head_dim * float(last["lq"].sum()),
                    "kernel_ms": bwd_ms, "fwd_kernel": fwd_part, "frac_of_nominal_2250": achieved / 2250.0}

    if args.norms:
        # the two row-norm kernels alone against the HBM roofline: each reads and writes one bf16 [T, H, D] tensor
        x = last["q"].detach()
        sumsq = torch.ones(x.shape[0], dtype=torch.float32, device=dev)
        nbytes = 2.0 * x.numel() * x.element_size()
        hbm = peaks["hbm_gbs"]
        norm_part = {}
        for name, fn in (("gdpa_layernorm_rows_kernel", lambda: G.layernorm_rows(x)),
                         ("gdpa_rmsnorm_rows_kernel", lambda: G.rmsnorm_rows(x, row_sumsq=sumsq))):
            for _ in range(3):
                fn()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                fn()
            b_.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b_) / 10
            norm_part[name] = {"bound": "hbm", "kernel_ms": ms, "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": hbm,
                               "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / hbm, "algorithmic_bytes": nbytes,
                               "note": "timed with the output allocation of the Python wrapper inside the loop"}
        roofline["norm_kernels"] = norm_part

    # ---- end to end: pinned host buffers, H2D of the inputs and D2H of every result per step ----
    e2e = None
    if not args.no_e2e and not strong and not fwd_only:
        b = batches[0]
        host_in = {n: b[n].detach().cpu().pin_memory() for n in ("q", "k", "v", "do")}
        host_out = {n: torch.empty_like(host_in["q" if n in ("o", "dq") else "k"]).pin_memory() for n in ("o", "dq", "dk", "dv")}
        h2d = sum(x.numel() * x.element_size() for x in host_in.values())
        d2h = sum(x.numel() * x.element_size() for x in host_out.values())

        host_off = {"q": b["q_offsets"].cpu(), "k": b["kv_offsets"].cpu()}

        def e2e_step():
            # public host-buffer entry point: token-balanced chunks, copies overlapped with the kernels
            G.forward_backward_host(host_in["q"], host_in["k"], host_in["v"], host_in["do"], host_off["q"], host_off["k"],
                                    qk_scale=w.qk_scale, activation=w.activation, out=host_out, n_chunks=args.e2e_chunks,
                                    device=dev)

        e2e_step()
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        a1.record()
        barrier()
        te = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item()) / args.e2e_steps
        e2e = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": args.e2e_steps,
               "api": "gdpa.forward_backward_host (pinned host Q, K, V, dO in; O, dQ, dK, dV out; %d chunks, copies overlapped with compute)" % args.e2e_chunks}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, dt, cores, sample = _cpu_oracle_rate(DEFAULT_WORKLOAD if (strong or fwd_only) else args.workload)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3" if fp8 else ("mxfp8 in, bf16 contraction" if mx else "bf16"), "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": int(sum(len(b["lq"]) for b in batches)), "heads": w.heads,
                       "head_dim": w.head_dim, "activation": w.activation, "pass": ("fwd+norms" if args.norms else "fwd") if fwd_only else "fwd+bwd",
                       "tokens_per_step": int(total_tokens), "useful_tflop_per_step": total_flops / 1e12,
                       "l2": "inputs larger than L2 (each of Q, K, V, dO exceeds 126 MB), no flush",
                       "parallelism": f"batch sharded by sequence over {world} GPU(s), no collective"},
            "per_gpu_tflops": value / world, "frac_of_nominal_bf16_peak": value / world / 2250.0,
            "frac_of_measured_bf16_sustained": value / world / peak,
            "tokens_per_s": total_tokens / (ms_step * 1e-3),
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
