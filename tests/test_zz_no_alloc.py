"""The allocation-free forward entry point, gdpa_fwd_noalloc, called through the C ABI.

Some hosts of this library cannot allocate device memory for the work schedule the ordinary forward
needs (a server whose arena owns the whole GPU, code running where an allocation would stall the
device).  For them the schedule lives in a fixed array inside the library.  The test checks that the
entry point gives the same output as gdpa_fwd on two calls in a row with different batches (the
array keeps the first call's contents, which must not leak into the second), and that a batch beyond
the stated limit is refused.  This file is collected last so that a run stopping at the first
failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests._util import ATOL, RTOL, assert_close, jagged_inputs

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


def test_noalloc_forward_matches_regular_forward_twice_in_a_row():
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi
    from ads_model_kernel_library_b200.gdpa import ops

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = [
        ([300, 70, 513, 129], [260, 200, 700, 131], 4, 128, 2, 1.0 / 64),   # gelu_approx
        ([40, 1000, 17], [90, 333, 512], 2, 64, 7, 1.0 / 32),               # silu, fewer items than before
    ]
    for lq, lk, H, D, act_id, scale in cases:
        cpu, dev = jagged_inputs(lq, lk, H, D, seed=21, std=0.5)
        # existing entry point, with a caller-allocated schedule
        sched = ops._build_schedule(cabi.GDPA_SCHED_FWD, dev["qo"], dev["ko"], len(lq), H, dev["q"].shape[0],
                                    int(max(lq)), int(max(lk)))
        o_ref = torch.zeros_like(dev["q"])
        cabi.check(cabi.lib.gdpa_fwd(C.byref(_params(cabi, dev, lq, lk, H, D, act_id, scale, o_ref, sched)), stream), "gdpa_fwd")
        # new entry point: inputs and outputs only
        o_new = torch.zeros_like(dev["q"])
        cabi.check(cabi.lib.gdpa_fwd_noalloc(C.byref(_params(cabi, dev, lq, lk, H, D, act_id, scale, o_new, None)), stream),
                   "gdpa_fwd_noalloc")
        torch.cuda.synchronize()
        assert_close(o_new, o_ref.float(), "O (no-alloc vs regular)", atol=ATOL, rtol=RTOL)
        assert torch.equal(o_new, o_ref)  # same kernel, same tiles: bitwise equal as well


def test_noalloc_rejects_batches_beyond_its_limit():
    from ads_model_kernel_library_b200.gdpa import _cabi as cabi

    p = cabi.GdpaFwdParams()
    p.struct_size = C.sizeof(cabi.GdpaFwdParams)
    p.heads, p.head_dim, p.batch = 8, 128, 10000   # 8 * 10000 items > 65536
    p.total_q = 10000
    rc = cabi.lib.gdpa_fwd_noalloc(C.byref(p), None)
    assert rc == 10
    assert b"GDPA_NOALLOC_MAX_ITEMS" in cabi.lib.gdpa_strerror(rc)
