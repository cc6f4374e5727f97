"""CPU-only tests: the C-ABI library loads and exports every declared symbol, argument checks of
the entry points that run before any CUDA call, host-side helpers (shard planner, workloads)."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cabi():
    from ads_model_kernel_library_b200.gdpa import _cabi

    return _cabi


def test_library_exports_every_symbol_the_header_declares(cabi):
    hdr = open(os.path.join(ROOT, "include", "gdpa_b200.h")).read()
    declared = set(re.findall(r"^\s*(?:int|size_t|const char\*|int64_t|int32_t|void)\s+(gdpa_\w+)\s*\(", hdr, re.M))
    assert declared, "no declarations parsed"
    assert declared == set(cabi.EXPORTS)
    for name in declared:
        assert hasattr(cabi.lib, name), name
    assert cabi.lib.gdpa_version() >= 100
    assert cabi.lib.gdpa_strerror(0) == b"ok"


def test_struct_sizes_match_between_python_and_c(cabi):
    # a mismatching struct_size is rejected, a matching one passes on to the next check
    p = cabi.GdpaFwdParams()
    p.struct_size = 4
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 1
    p.struct_size = C.sizeof(cabi.GdpaFwdParams)
    p.heads, p.head_dim = 2, 96
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 2  # unsupported head_dim: struct layout agreed
    b = cabi.GdpaBwdParams()
    b.struct_size = C.sizeof(cabi.GdpaBwdParams)
    b.heads, b.head_dim = 2, 32
    assert cabi.lib.gdpa_bwd(C.byref(b), None) == 2
    s = cabi.GdpaSchedParams()
    s.struct_size = C.sizeof(cabi.GdpaSchedParams) - 1
    assert cabi.lib.gdpa_build_schedule(C.byref(s), None) == 1


def test_argument_checks_before_any_cuda_call(cabi):
    p = cabi.GdpaFwdParams()
    p.struct_size = C.sizeof(cabi.GdpaFwdParams)
    p.heads, p.head_dim, p.batch = 2, 128, 1
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 1  # null offsets / schedule
    p.q_offsets = p.kv_offsets = p.schedule = 16
    p.activation = 55
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 4  # unknown activation
    p.activation = 2
    p.dtype = 7
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 3  # unsupported dtype
    p.dtype = 0
    p.total_q = 1 << 31
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 1  # row index beyond 32 bits
    p.total_q = 0
    assert cabi.lib.gdpa_fwd(C.byref(p), None) == 0  # nothing to do
    assert b"head_dim" in cabi.lib.gdpa_strerror(2)


def test_mxfp8_entry_points_check_arguments_before_any_cuda_call(cabi):
    for fn in (cabi.lib.gdpa_quantize_mxfp8, cabi.lib.gdpa_dequantize_mxfp8):
        p = cabi.GdpaMxParams()
        p.struct_size = 8
        assert fn(C.byref(p), None) == 1  # struct layout disagrees
        p.struct_size = C.sizeof(cabi.GdpaMxParams)
        p.heads, p.head_dim, p.batch, p.total = 2, 48, 1, 4
        p.offsets = p.block_offsets = 16
        assert fn(C.byref(p), None) == 1  # head_dim not a multiple of 32
        p.head_dim = 1024
        assert fn(C.byref(p), None) == 1  # more than four scale atoms per row
        p.head_dim, p.scale_axis = 128, 2
        assert fn(C.byref(p), None) == 1  # unknown scale axis
        p.scale_axis = 1
        assert fn(C.byref(p), None) == 1  # null data with total > 0
        p.x, p.x8, p.sf, p.sf_blocks = 16, 32, 52, 1
        assert fn(C.byref(p), None) == 5  # GDPA_ERR_MISALIGNED: scale tensor not 16-byte aligned
        p.sf, p.total, p.sf_blocks = 64, 300, 2
        assert fn(C.byref(p), None) == 8  # GDPA_ERR_CAPACITY: 300 rows need at least three blocks of scales


def test_schedule_and_workspace_sizes(cabi):
    lib = cabi.lib
    assert lib.gdpa_schedule_bytes(0, 1000, 4, 2) == 16 + 16 * 2 * (1000 // 256 + 4)
    assert lib.gdpa_schedule_bytes(1, 1000, 4, 2) == 16 + 16 * 2 * (1000 // 128 + 4)
    assert lib.gdpa_bwd_workspace_bytes(10, 2, 64) == 10 * 2 * 64 * 4
    assert lib.gdpa_schedule_bytes(0, -1, 4, 2) == 0


def test_operator_has_no_cpu_path():
    import ads_model_kernel_library_b200.gdpa as G

    q = torch.zeros(4, 1, 64, dtype=torch.bfloat16)
    off = torch.tensor([0, 4])
    with pytest.raises((NotImplementedError, RuntimeError)):
        G.generalized_dot_product_attention(q, q, q, off, off, 4, 4, activation="relu")


def test_activation_table_mirrors_reference_names():
    import json

    import ads_model_kernel_library_b200.gdpa as G

    ids = json.load(open(os.path.join(ROOT, "tests", "golden", "activation_ids.json")))
    for name, i in ids.items():
        assert G.activation_string_to_int(name) == i
    assert G.activation_string_to_int("softmax") == 100
    with pytest.raises(ValueError):
        G.activation_string_to_int("tanh")


def test_unsupported_options_raise_like_the_reference():
    import ads_model_kernel_library_b200.gdpa as G

    q = torch.zeros(4, 1, 64, dtype=torch.bfloat16)
    off = torch.tensor([0, 4])
    with pytest.raises(NotImplementedError):
        G.generalized_dot_product_attention(q, q, q, off, off, 4, 4, attn_mask=torch.zeros(1))
    with pytest.raises(NotImplementedError):
        G.generalized_dot_product_attention(q, q, q, off, off, 4, 4, window_size=3)
    with pytest.raises(ValueError):  # a fused QKV tensor needs a last dimension of 3 * head_dim
        G.generalized_dot_product_attention(q, None, None, off, off, 4, 4)
    with pytest.raises(ValueError):
        G.generalized_dot_product_attention(q, None, q, off, off, 4, 4)


def test_token_balanced_shard_planner():
    from ads_model_kernel_library_b200.gdpa import plan_token_balanced_shards, shard_jagged
    from ads_model_kernel_library_b200.gdpa.workloads import make_workload

    w = make_workload("c5_zipf_sharded")
    for n in (1, 2, 4, 8):
        shards = plan_token_balanced_shards(w.q_lens, w.kv_lens, n)
        assert len(shards) == n and shards[0][0] == 0 and shards[-1][1] == len(w.q_lens)
        assert all(shards[i][1] == shards[i + 1][0] for i in range(n - 1))
        tok = [int((w.q_lens[s:e] + w.kv_lens[s:e]).sum()) for s, e in shards]
        assert max(tok) - min(tok) <= 2 * 2 * 8192  # within one longest sequence of each other
    # more shards than sequences
    shards = plan_token_balanced_shards([5, 5], [5, 5], 4)
    assert sum(e - s for s, e in shards) == 2
    off = np.array([0, 3, 10, 12])
    assert shard_jagged(off, 1, 3)[0:2] == (3, 12)
    assert list(shard_jagged(off, 1, 3)[2]) == [0, 7, 9]
    with pytest.raises(ValueError):
        plan_token_balanced_shards([1], [1, 2], 2)


def test_workload_generators_are_seeded_and_shaped():
    from ads_model_kernel_library_b200.gdpa.workloads import WORKLOADS, make_workload, useful_flops

    for name in WORKLOADS:
        a, b = make_workload(name), make_workload(name)
        assert (a.q_lens == b.q_lens).all() and (a.kv_lens == b.kv_lens).all()
    c3 = make_workload("c3_fwd_bwd_gelu_uniform")
    assert len(c3.q_lens) == 512 and c3.q_lens.min() >= 512 and c3.q_lens.max() <= 4096 and c3.heads == 8
    c5 = make_workload("c5_zipf_sharded")
    assert c5.q_lens.min() >= 32 and c5.q_lens.max() == 8192 and len(c5.q_lens) == 8192
    assert useful_flops([2], [3], 1, 64, "bwd") == 10 * 64 * 6


def test_flop_formula_counts_valid_pairs_only():
    from ads_model_kernel_library_b200.gdpa import ops

    qo, ko = torch.tensor([0, 3, 10]), torch.tensor([0, 5, 9])
    assert ops._valid_pairs(qo, ko, 100, 100) == 3 * 5 + 7 * 4
    assert ops._valid_pairs(qo, ko, 4, 100) == 3 * 5 + 4 * 4  # clamped to max_seq_len_q
    meta = torch.empty(3, device="meta", dtype=torch.int64)
    assert ops._valid_pairs(meta, meta, 8, 16) == 2 * 8 * 16


def test_clock_sampler_keeps_the_samples_of_the_timed_region_only():
    """bench.py starts nvidia-smi before the warm-up (its start-up can outlast a short timed region) and keeps the
    samples that arrive after the mark it takes when the timed region begins; the reported clock is the median of the
    samples under load."""
    import sys

    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench

    class Proc:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    s = bench.ClockSampler(0)
    s.proc = Proc()
    idle = "1965, 1965, 200.0, Not Active, Not Active, Not Active, Not Active"
    s.lines = [idle] * 3
    first = s.mark(0.0)
    assert first == 3
    s.lines += ["1500, 1965, 700.0, Not Active, Not Active, Not Active, Active", idle,
                "1520, 1965, 720.0, Not Active, Not Active, Not Active, Active"]
    out = s.stop(first)
    assert out["samples"] == 3 and out["samples_under_load"] == 2
    assert out["sm_mhz"] == 1510.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
    # no sample after the mark: the last one before it is kept rather than none
    s2 = bench.ClockSampler(0)
    s2.proc = Proc()
    s2.lines = [idle] * 2
    assert s2.stop(s2.mark(0.0))["samples"] == 1
