"""The allocation-free forward entry point, gdpa_fwd_noalloc, called through the C ABI.

Some hosts of this library cannot allocate device memory for the work schedule the ordinary forward
needs (a server whose arena owns the whole GPU, code running where an allocation would stall the
device).  For them the schedule lives in a fixed array inside the library.  The tests check that the
entry point gives the same output as gdpa_fwd -- and as the CPU oracle -- on calls in a row with
different batches (the array keeps the previous call's contents, which must not leak into the next),
that the calls leave the amount of free device memory unchanged, that a batch beyond the stated limit
is refused, and that a call gdpa_fwd would refuse is refused before the shared array is touched.  This
file is collected last so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests._util import ATOL, RTOL, assert_close, jagged_inputs, oracle_forward

pytestmark = pytest.mark.gpu


def _params(cabi, dev, lq, lk, H, D, act_id, scale, o, sched):
    p = cabi.GdpaFwdParams()
    p.struct_size = C.sizeof(cabi.GdpaFwdParams)
    p.dtype = cabi.GDPA_DTYPE_BF16
    p.q, p.k, p.v, p.o = dev["q"].data_ptr(), dev["k"].data_ptr(), dev["v"].data_ptr(), o.data_ptr()
    p.q_offsets, p.kv_offsets = dev["qo"].data_ptr(), dev["ko"].data_ptr()
    p.offsets_are_int64 = 1
    p.batch = len(lq)
    p.total_q, p.total_kv = dev["q"].shape[0], dev["k"].shape[0]
    p.heads, p.head_dim = H, D
    p.max_seq_len_q, p.max_seq_len_kv = int(max(lq)), int(max(lk))
    p.activation = act_id
    p.qk_scale = scale
    p.schedule = 0 if sched is None else sched.data_ptr()
    return p


ACT_NAMES = {2: "gelu_approx", 7: "silu", 100: "softmax"}


def test_noalloc_forward_matches_regular_forward_twice_in_a_row():
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi
    from ads_model_kernel_library_b200.gdpa import ops

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = [
        ([300, 70, 513, 129], [260, 200, 700, 131], 4, 128, 2, 1.0 / 64),   # gelu_approx
        ([40, 1000, 17], [90, 333, 512], 2, 64, 7, 1.0 / 32),               # silu, fewer items than before
        ([129, 5, 700], [64, 300, 257], 2, 128, 100, 0.125),                # softmax, with the log-sum-exp output
    ]
    # the first call on the device resolves the array's address; measure free memory over the calls after it
    for i, (lq, lk, H, D, act_id, scale) in enumerate(cases):
        cpu, dev = jagged_inputs(lq, lk, H, D, seed=21, std=0.5)
        # existing entry point, with a caller-allocated schedule
        sched = ops._build_schedule(cabi.GDPA_SCHED_FWD, dev["qo"], dev["ko"], len(lq), H, dev["q"].shape[0],
                                    int(max(lq)), int(max(lk)))
        o_ref = torch.zeros_like(dev["q"])
        o_new = torch.zeros_like(dev["q"])
        lse_ref = torch.zeros(H, dev["q"].shape[0], dtype=torch.float32, device="cuda")
        lse_new = torch.zeros_like(lse_ref)
        p_ref = _params(cabi, dev, lq, lk, H, D, act_id, scale, o_ref, sched)
        p_new = _params(cabi, dev, lq, lk, H, D, act_id, scale, o_new, None)
        if act_id == 100:
            p_ref.lse, p_new.lse = lse_ref.data_ptr(), lse_new.data_ptr()
        cabi.check(cabi.lib.gdpa_fwd(C.byref(p_ref), stream), "gdpa_fwd")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        # new entry point: inputs and outputs only
        cabi.check(cabi.lib.gdpa_fwd_noalloc(C.byref(p_new), stream), "gdpa_fwd_noalloc")
        torch.cuda.synchronize()
        if i > 0:
            assert torch.cuda.mem_get_info()[0] == free_before, "gdpa_fwd_noalloc changed the free device memory"
        assert_close(o_new, o_ref.float(), "O (no-alloc vs regular)", atol=ATOL, rtol=RTOL)
        assert torch.equal(o_new, o_ref)  # same kernel, same tiles: bitwise equal as well
        assert torch.equal(lse_new, lse_ref)
        assert_close(o_new, oracle_forward(cpu, ACT_NAMES[act_id], scale), "O (no-alloc vs oracle)", atol=ATOL, rtol=RTOL)


def test_noalloc_shared_kv_index():
    """Many Q sequences reading one KV sequence (kv_seq_index) through the allocation-free entry point."""
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi
    from ads_model_kernel_library_b200.gdpa import ops
    from oracle import gdpa_oracle as orc

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lq, lk, H, D = [50, 130, 7, 260], [200, 90], 2, 128
    cpu, dev = jagged_inputs(lq, [200, 90, 1, 1], H, D, seed=22, std=0.5)
    ko = torch.tensor([0, 200, 290], dtype=torch.int64)
    index = torch.tensor([1, 0, 0, 1], dtype=torch.int64)
    o = torch.zeros_like(dev["q"])
    p = _params(cabi, dev, lq, lk, H, D, 2, 1.0 / 64, o, None)
    ko_d, index_d = ko.cuda(), index.cuda()
    p.kv_offsets, p.kv_seq_index, p.kv_batch = ko_d.data_ptr(), index_d.data_ptr(), 2
    cabi.check(cabi.lib.gdpa_fwd_noalloc(C.byref(p), stream), "gdpa_fwd_noalloc")
    torch.cuda.synchronize()
    # oracle: gather each Q sequence's KV rows
    ks = [cpu["k"][int(ko[j]):int(ko[j + 1])] for j in index.tolist()]
    vs = [cpu["v"][int(ko[j]):int(ko[j + 1])] for j in index.tolist()]
    ko2 = torch.tensor(np.concatenate([[0], np.cumsum([x.shape[0] for x in ks])]))
    ref = orc.gdpa_forward(cpu["q"].float(), torch.cat(ks).float(), torch.cat(vs).float(), cpu["qo"], ko2, "gelu_approx", 1.0 / 64)
    assert_close(o, ref, "O (no-alloc, shared KV)")


def test_noalloc_refuses_what_gdpa_fwd_refuses_without_touching_the_array():
    """A call with an unsupported head_dim, dtype or activation, or a null Q, returns gdpa_fwd's error code and
    launches nothing (the launch counter does not move), so the shared array still holds the last good schedule."""
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lq, lk = [100, 37], [64, 200]
    cpu, dev = jagged_inputs(lq, lk, 2, 64, seed=23, std=0.5)
    o = torch.zeros_like(dev["q"])
    good = _params(cabi, dev, lq, lk, 2, 64, 7, 0.1, o, None)
    n0 = cabi.lib.gdpa_launch_count()
    for field, value, code in (("head_dim", 96, 2), ("dtype", 1, 3), ("activation", 55, 4), ("q", 0, 1)):
        bad = _params(cabi, dev, lq, lk, 2, 64, 7, 0.1, o, None)
        setattr(bad, field, value)
        assert cabi.lib.gdpa_fwd_noalloc(C.byref(bad), stream) == code
    assert cabi.lib.gdpa_launch_count() == n0
    cabi.check(cabi.lib.gdpa_fwd_noalloc(C.byref(good), stream), "gdpa_fwd_noalloc")
    torch.cuda.synchronize()
    assert_close(o, oracle_forward(cpu, "silu", 0.1), "O after refused calls")


def test_noalloc_rejects_batches_beyond_its_limit():
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi

    lq, lk = [100, 37], [64, 200]
    cpu, dev = jagged_inputs(lq, lk, 8, 128, seed=24, std=0.5)
    p = _params(cabi, dev, lq, lk, 8, 128, 2, 0.1, torch.zeros_like(dev["q"]), None)
    p.batch = 10000  # 8 heads * 10000 sequences > 65536 items; refused on the host, nothing reads the short offset arrays
    n0 = cabi.lib.gdpa_launch_count()
    rc = cabi.lib.gdpa_fwd_noalloc(C.byref(p), None)
    assert rc == 10 and cabi.lib.gdpa_launch_count() == n0
    assert b"GDPA_NOALLOC_MAX_ITEMS" in cabi.lib.gdpa_strerror(rc)
