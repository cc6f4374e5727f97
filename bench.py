#!/usr/bin/env python
"""Benchmark of the GDPA hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one forward + backward pass of the operator over one jagged batch of synthetic input
(seeded; shapes and value distributions of the named workload).  The default workload is the
fwd+bwd BF16 configuration: B=512 sequences, H=8, D=128, Q=KV lengths uniform in [512, 4096],
GELU-tanh, scale 1/max_len, values N(0, 0.5).  With N > 1 (launched by torch.distributed.run, one
process per GPU) every rank runs its own batch of that configuration (weak scaling; sequences are
independent, so there is no collective on the data path) and the time is the maximum over ranks.

The default run additionally measures, at every N, the sharded configuration (B=8192 sequences, H=4,
D=128, Zipf(1.2) lengths 32 ... 8192, fwd+bwd) split over the N ranks by token-balanced offsets (strong
scaling): the JSON line's `strong_c5` object holds its whole-job TFLOP/s, the per-rank milliseconds
(the imbalance) and the same for a split balanced on sum(Lq * Lkv).  `--workload c5_zipf_sharded`
makes that configuration the line's `value`.

Rank 0 prints ONE JSON line.  `value` is whole-job useful TFLOP/s (14 H D sum(Lq Lkv) per step,
valid jagged pairs only) with the inputs resident in HBM; `e2e` is the same metric through the
public Python entry point with pinned HOST buffers, host<->device copies inside the timed region.
`--impl reference` times the reference's eager PyTorch formulation (the CPU oracle port) on the
host cores instead, on a fixed sample of the workload.

`--ref-grid` runs the workload of the reference's own published plots (gdpa/scripts/benchmark.py:176-185,
:574-598 of the reference: B=1152, H=4, D=128, fast_gelu, N(0,1) values, scale 1; self-attention with every Q
length at L or uniform in [1, L], cross-attention with KV fixed at 256; L in 256 ... 2048), forward and
backward timed separately at operator level, one JSON line per cell.
"""
from __future__ import annotations

import argparse
import ctypes
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
# 48 sequences of the default workload, H=8, D=128, with the kernels of commit e5537c8).  Traffic grows in
# proportion to the tokens, so a full launch is this figure times its Q tokens.
NCU_DRAM_BYTES_PER_TOKEN = {"gdpa_bwd_kernel": 2.323e9 / 114351, "gdpa_fwd_kernel": 0.929e9 / 114351}

METRIC = "gdpa_fwd_bwd_useful_tflops"
UNIT = "TFLOP/s"
DEFAULT_WORKLOAD = "c3_fwd_bwd_gelu_uniform"
# The CPU legs (`cpu_baseline` of a normal run and every step of `--impl reference`) time the same fixed
# sample: the first sequences of the default workload, whatever --steps says.
CPU_SAMPLE_WORKLOAD = DEFAULT_WORKLOAD
CPU_SAMPLE_SEQUENCES = 8


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
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self, wait_s: float = 3.0) -> int:
        """Waits (bounded) until nvidia-smi has delivered its first sample -- its start-up can take longer than a short
        timed region -- and returns the number of samples so far: `stop(first=...)` then keeps only later ones."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < wait_s:
            time.sleep(0.02)
        return len(self.lines)

    def stop(self, first: int = 0):
        self.lines = self.lines[first:] if first < len(self.lines) else self.lines[-1:]
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
        # under load = samples drawing more than half of the highest power seen (the sampler also runs while
        # the host prepares the next launch)
        load = [s for s, p in zip(sm, pw) if p >= 0.5 * max(pw)]
        return {"sm_mhz": float(np.median(load if load else sm)), "sm_max_mhz": float(max(mx)), "power_w_max": float(max(pw)),
                "samples": len(sm), "samples_under_load": len(load), "reasons": sorted(reasons)}


def _gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


# ------------------------------------------------------------------------------------------------
# Host placement: a rank's pinned buffers should live on the NUMA node its GPU hangs off.
# ------------------------------------------------------------------------------------------------
def bind_host_to_gpu_node(local_rank: int) -> dict:
    """Best effort, before any pinned allocation: restrict this process to the CPUs of the NUMA node of its GPU
    and prefer that node for its memory (set_mempolicy).  Returns what was found and done; on hosts that expose
    one node, or whose container may not leave its CPU set, this changes nothing and says so."""
    info = {"cpus_allowed": len(os.sched_getaffinity(0)), "bound": False}
    try:
        out = subprocess.run(["nvidia-smi", "-i", str(_gpu_index(local_rank)), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip()
        pci = out.lower().replace("00000000:", "0000:") if out else None
        node_path = f"/sys/bus/pci/devices/{pci}/numa_node" if pci else None
        node = int(open(node_path).read()) if node_path and os.path.exists(node_path) else -1
        nodes = sorted(int(d[4:]) for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit())
        info.update(gpu_numa_node=node, host_numa_nodes=len(nodes))
        if node < 0 or len(nodes) < 2:
            info["note"] = "one NUMA node visible (or the GPU reports none): nothing to bind"
            return info
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        usable = cpus & os.sched_getaffinity(0)
        if not usable:
            info["note"] = f"the CPUs of node {node} are outside this process's allowed set: left unbound"
            return info
        os.sched_setaffinity(0, usable)
        libc = ctypes.CDLL(None, use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        MPOL_PREFERRED, SYS_set_mempolicy = 1, 238  # x86-64 syscall number
        rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64))
        info.update(bound=True, cpus_bound=len(usable), mempolicy_rc=int(rc))
    except Exception as exc:  # placement is an optimisation, never a reason to fail the benchmark
        info["note"] = f"placement probe failed: {type(exc).__name__}: {exc}"
    return info


# ------------------------------------------------------------------------------------------------
# CPU legs
# ------------------------------------------------------------------------------------------------
_cpu_sample_cache = {}


def _cpu_sample():
    """The fixed CPU sample: the first CPU_SAMPLE_SEQUENCES sequences of the default workload, N(0, 0.5) values."""
    if not _cpu_sample_cache:
        from ads_model_kernel_library_b200.gdpa.workloads import make_workload, useful_flops

        w = make_workload(CPU_SAMPLE_WORKLOAD)
        n = CPU_SAMPLE_SEQUENCES
        lq, lk = w.q_lens[:n], w.kv_lens[:n]
        qo = torch.from_numpy(np.concatenate([[0], np.cumsum(lq)]))
        ko = torch.from_numpy(np.concatenate([[0], np.cumsum(lk)]))
        g = torch.Generator().manual_seed(0)
        t = {name: torch.randn(int(off[-1]), w.heads, w.head_dim, generator=g) * w.std
             for name, off in (("q", qo), ("k", ko), ("v", ko), ("do", qo))}
        _cpu_sample_cache.update(w=w, qo=qo, ko=ko, t=t, flops=useful_flops(lq, lk, w.heads, w.head_dim, "fwd_bwd"),
                                 text=f"first {n} sequences of {CPU_SAMPLE_WORKLOAD} ({int(qo[-1])} Q tokens), fwd+bwd fp32 eager")
    return _cpu_sample_cache


def _cpu_oracle_rate():
    """Useful TFLOP/s of the eager fp32 formulation (the oracle port) on all host cores over the fixed sample."""
    from oracle import gdpa_oracle as orc

    s = _cpu_sample()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w, t = s["w"], s["t"]
    t0 = time.perf_counter()
    orc.gdpa_forward_backward(t["q"], t["k"], t["v"], s["qo"], s["ko"], t["do"], w.activation, w.qk_scale)
    dt = time.perf_counter() - t0
    return s["flops"] / dt / 1e12, dt, cores, f"{s['text']}, {dt:.1f} s, {torch.get_num_threads()} torch threads"


def run_reference(args, rank: int):
    """The reference arm: the reference's own CPU formulation of the path (eager PyTorch fp32 per
    sequence, autograd backward) on all host cores, same metric; every step is the fixed sample."""
    if rank != 0:
        return
    from ads_model_kernel_library_b200.gdpa.workloads import make_workload

    w = make_workload(args.workload)
    vals, dts = [], []
    sample = ""
    for i in range(args.warmup + args.steps):
        v, dt, cores, sample = _cpu_oracle_rate()
        if i >= args.warmup:
            vals.append(v); dts.append(dt)
    value = float(np.mean(vals))
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.mean(dts) * 1e3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": int(len(w.q_lens)), "heads": w.heads, "head_dim": w.head_dim,
                   "activation": w.activation, "pass": "fwd+bwd", "sampled": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count() or 1, "torch_threads": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# The sharded Zipf configuration: token-balanced (and pair-balanced) split over the ranks, strong scaling
# ------------------------------------------------------------------------------------------------
def run_strong_c5(G, dev, rank: int, world: int, dist, peaks, steps: int, warmup: int, balances=("tokens", "pairs"),
                  batch=None, sampler_index=None):
    """One entry per balance mode: whole-job TFLOP/s with time = max over ranks, and every rank's own time.
    A rank's sequence range comes from the planner; on fewer than 8 GPUs the range is run as several pieces, one
    after another, so that the outputs and the fp32 dQ accumulator of one piece at a time fit beside the inputs."""
    from ads_model_kernel_library_b200.gdpa.sharding import gather_rows, plan_token_balanced_shards
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload, useful_flops

    w = make_workload("c5_zipf_sharded", batch=batch)
    result = {"workload": "c5_zipf_sharded", "batch": int(len(w.q_lens)), "heads": w.heads, "head_dim": w.head_dim,
              "activation": w.activation, "pass": "fwd+bwd", "steps": steps, "warmup": warmup, "scaling": "strong"}
    pieces_per_rank = max(1, 8 // world)
    if world == 1:
        balances = balances[:1]  # one rank: the split does not matter
    sampler = ClockSampler(sampler_index).start() if (rank == 0 and sampler_index is not None) else None
    for balance in balances:
        s, e = plan_token_balanced_shards(w.q_lens, w.kv_lens, world, balance)[rank]
        sub = plan_token_balanced_shards(w.q_lens[s:e], w.kv_lens[s:e], pieces_per_rank)
        batches = []
        for i, (a, b) in enumerate(sub):
            if b <= a:
                continue
            t = make_tensors(w, dev, seed=5000 + 1000 * rank + i, with_grad_out=True, seq_range=(s + a, s + b))
            t["lq"], t["lk"] = w.q_lens[s + a:s + b], w.kv_lens[s + a:s + b]
            t["max_q"], t["max_kv"] = int(t["lq"].max()), int(t["lk"].max())
            batches.append(t)
        flops_rank = sum(useful_flops(b["lq"], b["lk"], w.heads, w.head_dim, "fwd_bwd") for b in batches)
        tokens_rank = sum(int(b["lq"].sum() + b["lk"].sum()) for b in batches)

        def step():
            for b in batches:
                q, k, v = b["q"].requires_grad_(True), b["k"].requires_grad_(True), b["v"].requires_grad_(True)
                o = G.generalized_dot_product_attention(q, k, v, b["q_offsets"], b["kv_offsets"], b["max_q"], b["max_kv"],
                                                        qk_scale=w.qk_scale, activation=w.activation)
                o.backward(b["do"])
                q.grad = k.grad = v.grad = None
                del o

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(warmup):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        assert G.kernel_status() == 0, "a kernel wait ran out in the sharded configuration"
        mine = torch.tensor([e0.elapsed_time(e1) / steps, float(flops_rank), float(tokens_rank)], dtype=torch.float64, device=dev)
        if world > 1:
            allr = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
        else:
            allr = [mine]
        per_rank_ms = [float(x[0]) for x in allr]
        total_flops = sum(float(x[1]) for x in allr)
        total_tokens = sum(float(x[2]) for x in allr)
        ms = max(per_rank_ms)
        tfl = total_flops / (ms * 1e-3) / 1e12
        result[balance] = {"value": tfl, "unit": UNIT, "ms_per_step": ms, "per_rank_ms": per_rank_ms,
                           "per_rank_tflop": [float(x[1]) / 1e12 for x in allr],
                           "imbalance_max_over_mean": ms / (sum(per_rank_ms) / len(per_rank_ms)),
                           "tokens_per_s": total_tokens / (ms * 1e-3), "per_gpu_tflops": tfl / world,
                           "frac_of_measured_bf16_sustained": tfl / world / peaks["bf16_tflops_sustained"],
                           "frac_of_nominal_bf16_peak": tfl / world / 2250.0, "pieces_per_rank": len(batches)}
        if balance == balances[0]:
            # validation, the one use of a collective: every rank runs the forward on the first sequences of its
            # range, the O shards are gathered in rank order, and rank 0 recomputes them all from the seeds
            nv = 4
            def small(r):
                rs, _ = plan_token_balanced_shards(w.q_lens, w.kv_lens, world, balance)[r]
                t = make_tensors(w, dev, seed=777 + r, seq_range=(rs, rs + nv))
                with torch.no_grad():
                    return G.generalized_dot_product_attention(t["q"], t["k"], t["v"], t["q_offsets"], t["kv_offsets"],
                                                               int(w.q_lens[rs:rs + nv].max()), int(w.kv_lens[rs:rs + nv].max()),
                                                               qk_scale=w.qk_scale, activation=w.activation)
            o_mine = small(rank)
            gathered = gather_rows(o_mine) if world > 1 else o_mine
            if rank == 0:
                expect = torch.cat([small(r) for r in range(world)])
                result["gathered_shards_match_recomputation"] = bool(torch.equal(gathered, expect))
                result["gathered_rows"] = int(gathered.shape[0])
        del batches
        torch.cuda.empty_cache()
    if sampler is not None:
        result["clocks"] = sampler.stop()
    if "pairs" in result and "tokens" in result:
        result["better_split"] = "pairs" if result["pairs"]["value"] > result["tokens"]["value"] else "tokens"
    return result


# ------------------------------------------------------------------------------------------------
# The reference's published workload, cell by cell
# ------------------------------------------------------------------------------------------------
REF_SETS = {"self_s1": "self-attention, every Q length = L, KV = L", "self_s05": "self-attention, Q length uniform in [1, L], KV = L",
            "cross_kv256": "cross-attention, Q length = L, KV = 256"}
# TFLOP/s read off the bar charts of the reference's README (B200 at 750 W, its CuteDSL kernel), fwd / bwd at L = 256 ... 2048
REF_PUBLISHED = {("self_s1", "fwd"): (815, 900, 1015, 1145), ("self_s1", "bwd"): (255, 410, 570, 705),
                 ("self_s05", "fwd"): (500, 610, 795, 985), ("self_s05", "bwd"): (160, 270, 420, 580),
                 ("cross_kv256", "fwd"): (810, 825, 775, 785), ("cross_kv256", "bwd"): (258, 342, 408, 455)}
REF_LENGTHS = (256, 512, 1024, 2048)


def _ref_cell_lengths(kind: str, L: int, B: int, rng):
    """Lengths as the reference's generator draws them (gdpa/utils/utils.py:86-99): sparsity 1.0 -> every Q length L,
    0.5 -> uniform in [1, L]; K / V dense with `dff` rows per sequence."""
    if kind == "self_s05":
        lq = rng.integers(1, L + 1, B)
    else:
        lq = np.full(B, L, dtype=np.int64)
    lk = np.full(B, 256 if kind == "cross_kv256" else L, dtype=np.int64)
    return lq.astype(np.int64), lk


def run_ref_grid(args):
    """Forward and backward of every cell of the reference's published plots, each timed on its own at operator
    level (CUDA events around the whole op: schedule build, kernels, dQ rounding), median of the timed calls."""
    import ads_model_kernel_library_b200.gdpa as G
    from ads_model_kernel_library_b200.gdpa.math import activation_string_to_int
    from ads_model_kernel_library_b200.gdpa.workloads import useful_flops

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, H, D, act = args.batch or 1152, 4, 128, "fast_gelu"
    act_id = activation_string_to_int(act)
    peaks = _peaks()
    kinds = args.ref_sets.split(",") if args.ref_sets else list(REF_SETS)
    for kind in kinds:
        for li, L in enumerate(REF_LENGTHS):
            if args.ref_lengths and str(L) not in args.ref_lengths.split(","):
                continue
            rng = np.random.default_rng(2025 + L)
            lq, lk = _ref_cell_lengths(kind, L, B, rng)
            qo = torch.from_numpy(np.concatenate([[0], np.cumsum(lq)])).to(dev)
            ko = torch.from_numpy(np.concatenate([[0], np.cumsum(lk)])).to(dev)
            g = torch.Generator(device=dev).manual_seed(L)
            q, do = (torch.randn(int(lq.sum()), H, D, generator=g, device=dev).to(torch.bfloat16) for _ in range(2))
            k, v = (torch.randn(int(lk.sum()), H, D, generator=g, device=dev).to(torch.bfloat16) for _ in range(2))
            mq, mk = int(lq.max()), int(lk.max())
            calls = {
                "fwd": lambda: torch.ops.gdpa.generalized_dot_product_attention(q, k, v, qo, ko, mq, mk, 1.0, act_id),
                "bwd": lambda: torch.ops.gdpa.generalized_dot_product_attention_backward(do, q, k, v, qo, ko, mq, mk, 1.0, act_id),
            }
            for mode, fn in calls.items():
                flops = useful_flops(lq, lk, H, D, mode)
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); fn(); b.record(); torch.cuda.synchronize()
                reps = int(min(200, max(5, args.cell_ms / max(a.elapsed_time(b), 1e-3))))
                evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
                kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
                sampler = ClockSampler(_gpu_index(0)).start()
                for (x, y), k_ in zip(evs, kev):
                    with G.kernel_timing(**{mode: k_}):
                        x.record(); fn(); y.record()
                torch.cuda.synchronize()
                clocks = sampler.stop()
                assert G.kernel_status() == 0
                ms = float(np.median([x.elapsed_time(y) for x, y in evs]))
                kernel_ms = float(np.median([x.elapsed_time(y) for x, y in kev]))
                tfl = flops / (ms * 1e-3) / 1e12
                print(json.dumps({
                    "metric": f"gdpa_{mode}_useful_tflops", "value": tfl, "unit": UNIT, "n_gpus": 1, "steps": reps, "warmup": 3,
                    "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": f"ref_{kind}_{mode}_L{L}", "what": REF_SETS[kind], "batch": B, "heads": H, "head_dim": D,
                               "activation": act, "qk_scale": 1.0, "pass": mode, "q_tokens": int(lq.sum()), "kv_tokens": int(lk.sum()),
                               "l2": "inputs larger than L2, no flush", "timed": "operator level: schedule build, kernels, dQ rounding"},
                    "main_kernel_only": {"ms": kernel_ms, "value": flops / (kernel_ms * 1e-3) / 1e12, "unit": UNIT,
                                         "note": "the main kernel alone, without the schedule build (the reference's benchmark "
                                                 "builds its tile maps outside the timed call) and, backward, the accumulator "
                                                 "clear and the dQ rounding pass"},
                    "reference_published_tflops": REF_PUBLISHED[(kind, mode)][li],
                    "ratio_to_published": tfl / REF_PUBLISHED[(kind, mode)][li],
                    "frac_of_measured_bf16_sustained": tfl / peaks["bf16_tflops_sustained"], "frac_of_nominal_bf16_peak": tfl / 2250.0,
                    "clocks": clocks}), flush=True)
            del q, k, v, do
            torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the number of sequences (reduced-size runs)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunks", type=int, default=32)
    ap.add_argument("--activation", default=None, help="override the workload's activation (experiments)")
    ap.add_argument("--head-dim", type=int, default=None, help="override the workload's head_dim (64 or 128; profiling)")
    ap.add_argument("--norms", action="store_true",
                    help="time the forward of the GDPA-plus-norm pipeline (layer norm of Q, Q residual, RMS norm) "
                         "instead of the workload's own pass, and the two row-norm kernels against the HBM roofline")
    ap.add_argument("--mxfp8", action="store_true",
                    help="with --workload c4_fp8_softmax: feed the forward MXFP8 inputs (e4m3 + e8m0 scale per 32 elements); "
                         "the three de-quantising passes are inside the timed step")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the sharded Zipf configuration of the default run")
    ap.add_argument("--strong-steps", type=int, default=2)
    ap.add_argument("--strong-batch", type=int, default=None, help="sequences of the sharded configuration (reduced-size runs)")
    ap.add_argument("--ref-grid", action="store_true", help="run the reference's published workload cell by cell (one GPU)")
    ap.add_argument("--ref-sets", default=None, help="comma-separated subset of self_s1,self_s05,cross_kv256")
    ap.add_argument("--ref-lengths", default=None, help="--ref-grid: comma-separated subset of 256,512,1024,2048")
    ap.add_argument("--cell-ms", type=float, default=600.0, help="--ref-grid: milliseconds of timed calls per cell")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.ref_grid:
        if rank == 0:
            run_ref_grid(args)
        return

    if args.warmup < 3:
        args.warmup = 3
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    placement = bind_host_to_gpu_node(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import ads_model_kernel_library_b200.gdpa as G
    from ads_model_kernel_library_b200.gdpa import _cabi
    from ads_model_kernel_library_b200.gdpa.workloads import make_tensors, make_workload, useful_flops

    peaks = _peaks()
    peak = peaks["bf16_tflops_sustained"]
    strong = args.workload == "c5_zipf_sharded"
    if strong:
        # the sharded configuration as the headline of this run
        res = run_strong_c5(G, dev, rank, world, dist, peaks, steps=max(1, args.steps), warmup=args.warmup, batch=args.batch,
                            sampler_index=_gpu_index(local_rank))
        if rank == 0:
            best = res["tokens"]
            print(json.dumps({
                "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": best["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "batch": res["batch"], "heads": res["heads"], "head_dim": res["head_dim"],
                           "activation": res["activation"], "pass": "fwd+bwd", "split": "token-balanced contiguous sequence ranges",
                           "l2": "inputs larger than L2, no flush",
                           "parallelism": f"batch sharded by sequence over {world} GPU(s), no collective"},
                "per_gpu_tflops": best["per_gpu_tflops"], "frac_of_measured_bf16_sustained": best["frac_of_measured_bf16_sustained"],
                "tokens_per_s": best["tokens_per_s"], "strong_c5": res, "clocks": res.get("clocks"),
                "gpu_launches": int(_cabi.lib.gdpa_launch_count()), "roofline": None, "cpu_baseline": None, "e2e": None}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    w = make_workload(args.workload, batch=args.batch)
    if args.activation:
        w.activation = args.activation
    if args.head_dim:
        w.head_dim = args.head_dim
    fp8 = args.workload == "c4_fp8_softmax" and not args.mxfp8
    mx = args.workload == "c4_fp8_softmax" and args.mxfp8
    assert not args.mxfp8 or mx, "--mxfp8 goes with --workload c4_fp8_softmax"
    if args.norms:
        assert not fp8 and w.activation != "softmax", "--norms needs a bf16 workload with an element-wise activation"
        w.mode = "fwd"
    fwd_only = w.mode == "fwd"
    metric = METRIC if not fwd_only else ("gdpa_fwd_norms_useful_tflops" if args.norms else "gdpa_fwd_useful_tflops")
    t = make_tensors(w, dev, seed=1000 * rank, with_grad_out=True)
    t["lq"], t["lk"] = w.q_lens, w.kv_lens
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
    batches = [t]
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

    # the clock sampler starts before the warm-up, so that it is delivering samples when the timed region begins
    sampler = ClockSampler(_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    assert G.kernel_status() == 0, "a kernel wait ran out during warm-up"

    # ---- timed region: K steps, CUDA events on the launching stream, max over ranks ----------
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    bwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = _cabi.lib.gdpa_launch_count()
    first_sample = sampler.mark() if rank == 0 else 0
    barrier()
    e0.record()
    for i in range(args.steps):
        with G.kernel_timing(fwd=fwd_ev[i], bwd=bwd_ev[i]):
            step()
    e1.record()
    barrier()
    clocks = sampler.stop(first_sample) if rank == 0 else None
    launches = _cabi.lib.gdpa_launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    tt = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(flops_rank), float(tokens_rank)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_step = float(tt.item()) / args.steps
    total_flops, total_tokens = float(tot[0].item()), float(tot[1].item())
    value = total_flops / (ms_step * 1e-3) / 1e12
    assert G.kernel_status() == 0, "a kernel wait ran out during the timed region"

    # dominant kernel: the backward kernel (last call of each step carries the events)
    fwd_ms = float(np.mean([a.elapsed_time(b) for a, b in fwd_ev]))
    last = batches[-1]
    fwd_flops = useful_flops(last["lq"], last["lk"], w.heads, w.head_dim, "fwd")
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
                    "kernel_ms": bwd_ms, "fwd_kernel": fwd_part, "frac_of_nominal_2250": achieved / 2250.0,
                    "frac_of_measured_burst": achieved / peaks["bf16_tflops"]}

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
    if not args.no_e2e and not fwd_only:
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
        # every step between its own pair of events; the reported time is the median step (a host hiccup in one step --
        # these are seconds of host work on a shared machine -- does not decide the number), all steps are listed
        marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.e2e_steps)]
        for m0, m1 in marks:
            m0.record()
            e2e_step()
            m1.record()
        barrier()
        e2e_steps_ms = [m0.elapsed_time(m1) for m0, m1 in marks]
        # the host's ceiling: the same copies in the same chunks with no kernel between them
        dev_in = {n: torch.empty_like(b[n]) for n in ("q", "k", "v", "do")}
        rows = np.linspace(0, 1, args.e2e_chunks + 1)

        def copy_only():
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            for c in range(args.e2e_chunks):
                for (n_in, n_out) in (("q", "o"), ("do", "dq"), ("k", "dk"), ("v", "dv")):
                    r0, r1 = int(rows[c] * host_in[n_in].shape[0]), int(rows[c + 1] * host_in[n_in].shape[0])
                    with torch.cuda.stream(s_in):
                        dev_in[n_in][r0:r1].copy_(host_in[n_in][r0:r1], non_blocking=True)
                    with torch.cuda.stream(s_out):
                        host_out[n_out][r0:r1].copy_(dev_in[n_in][r0:r1], non_blocking=True)
            torch.cuda.current_stream().wait_stream(s_in)
            torch.cuda.current_stream().wait_stream(s_out)

        copy_only()
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        copy_only()
        c1.record()
        barrier()
        te = torch.tensor([float(np.median(e2e_steps_ms)), c0.elapsed_time(c1)], dtype=torch.float64, device=dev)
        if world > 1:
            all_te = [torch.zeros_like(te) for _ in range(world)]
            dist.all_gather(all_te, te)
        else:
            all_te = [te]
        e2e_ms = max(float(x[0]) for x in all_te)
        copy_ms = max(float(x[1]) for x in all_te)
        e2e = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": args.e2e_steps,
               "timed": "median step, max over ranks", "this_rank_steps_ms": [float(x) for x in e2e_steps_ms],
               "per_rank_ms": [float(x[0]) for x in all_te],
               "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
               "copy_only_ms_per_step": copy_ms, "copy_only_per_rank_ms": [float(x[1]) for x in all_te],
               "copy_only_gbs_each_way_per_rank": h2d / (copy_ms * 1e-3) / 1e9,
               "copy_only_note": "the same bytes in the same chunks, both directions at once, no kernels: the ceiling the host sets",
               "host_placement": placement,
               "api": "gdpa.forward_backward_host (pinned host Q, K, V, dO in; O, dQ, dK, dV out; %d chunks, copies overlapped with compute)" % args.e2e_chunks}
        del host_in, host_out, dev_in

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, dt, cores, sample = _cpu_oracle_rate()
        cpu_baseline = {"value": v, "unit": UNIT, "cores": cores, "torch_threads": torch.get_num_threads(), "kind": "port",
                        "sample": sample}

    strong_c5 = None
    if args.workload == DEFAULT_WORKLOAD and not args.no_strong and args.batch is None:
        t.clear()  # the one batch dictionary (also reachable as batches[0]): drop its tensors
        batches.clear()
        torch.cuda.empty_cache()
        strong_c5 = run_strong_c5(G, dev, rank, world, dist, peaks, steps=args.strong_steps, warmup=1, batch=args.strong_batch,
                                  sampler_index=_gpu_index(local_rank))

    if rank == 0:
        line = {
            "metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3" if fp8 else ("mxfp8 in, bf16 contraction" if mx else "bf16"), "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": int(len(w.q_lens)), "heads": w.heads,
                       "head_dim": w.head_dim, "activation": w.activation, "pass": ("fwd+norms" if args.norms else "fwd") if fwd_only else "fwd+bwd",
                       "tokens_per_step": int(total_tokens), "useful_tflop_per_step": total_flops / 1e12,
                       "l2": "inputs larger than L2 (each of Q, K, V, dO exceeds 126 MB), no flush",
                       "parallelism": f"batch sharded by sequence over {world} GPU(s), no collective"},
            "per_gpu_tflops": value / world, "frac_of_nominal_bf16_peak": value / world / 2250.0,
            "frac_of_measured_bf16_sustained": value / world / peak,
            "tokens_per_s": total_tokens / (ms_step * 1e-3),
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "strong_c5": strong_c5,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
