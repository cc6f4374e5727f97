"""ctypes binding of libgdpa_b200.so (C ABI declared in include/gdpa_b200.h).

The library is the only compute path of this package.  It is loaded on first use of ``_cabi.lib``
(so that host-only helpers such as the workload generators and the shard planner can be imported in a
process that never touches the GPU); if it is missing or cannot be loaded, that first use raises --
there is no fallback.  ``GDPA_B200_LIB`` overrides the path (a differently built copy of the library).
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("GDPA_B200_LIB") or os.path.join(_PKG, "libgdpa_b200.so")

# Return codes, activation ids and enums of include/gdpa_b200.h
GDPA_OK = 0
GDPA_DTYPE_BF16 = 0
GDPA_DTYPE_FP8_E4M3 = 1
GDPA_OFFSETS_INT64, GDPA_OFFSETS_PAIRS = 1, 2
GDPA_SCHED_FWD = 0
GDPA_SCHED_BWD = 1
GDPA_ACT_SOFTMAX = 100

EXPORTS = (
    "gdpa_schedule_bytes",
    "gdpa_build_schedule",
    "gdpa_fwd",
    "gdpa_fwd_fp8",
    "gdpa_fwd_noalloc",
    "gdpa_layernorm_rows",
    "gdpa_rmsnorm_rows",
    "gdpa_norm_rows_bwd",
    "gdpa_quantize_fp8_blockwise",
    "gdpa_quantize_mxfp8",
    "gdpa_dequantize_mxfp8",
    "gdpa_bwd_workspace_bytes",
    "gdpa_bwd",
    "gdpa_strerror",
    "gdpa_launch_count",
    "gdpa_version",
    "gdpa_debug_set_trace",
    "gdpa_debug_wait_probe",
)


class GdpaSchedParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("mode", C.c_int32),
        ("q_offsets", C.c_void_p),
        ("kv_offsets", C.c_void_p),
        ("offsets_are_int64", C.c_int32),
        ("batch", C.c_int32),
        ("heads", C.c_int32),
        ("max_seq_len_q", C.c_int32),
        ("max_seq_len_kv", C.c_int32),
        ("kv_batch", C.c_int32),
        ("schedule", C.c_void_p),
        ("schedule_bytes", C.c_int64),
        ("kv_seq_index", C.c_void_p),
    ]


class GdpaFwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("o", C.c_void_p),
        ("q_offsets", C.c_void_p),
        ("kv_offsets", C.c_void_p),
        ("offsets_are_int64", C.c_int32),
        ("batch", C.c_int32),
        ("total_q", C.c_int64),
        ("total_kv", C.c_int64),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("max_seq_len_q", C.c_int32),
        ("max_seq_len_kv", C.c_int32),
        ("activation", C.c_int32),
        ("qk_scale", C.c_float),
        ("schedule", C.c_void_p),
        ("status", C.c_void_p),
        ("q_scales", C.c_void_p),
        ("k_scales", C.c_void_p),
        ("v_scales", C.c_void_p),
        ("q_block_offsets", C.c_void_p),
        ("kv_block_offsets", C.c_void_p),
        ("timing_start_event", C.c_void_p),
        ("timing_stop_event", C.c_void_p),
        ("lse", C.c_void_p),
        ("kv_heads", C.c_int32),
        ("window_plus_one", C.c_int32),
        ("kv_seq_index", C.c_void_p),
        ("q_strides", C.c_int64 * 2),
        ("k_strides", C.c_int64 * 2),
        ("v_strides", C.c_int64 * 2),
        ("residual", C.c_void_p),
        ("row_sumsq", C.c_void_p),
        ("kv_batch", C.c_int32),
        ("reserved", C.c_int32),
    ]


class GdpaNormParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("n", C.c_int32),
        ("rows", C.c_int64),
        ("x", C.c_void_p),
        ("out", C.c_void_p),
        ("weight", C.c_void_p),
        ("bias", C.c_void_p),
        ("residual", C.c_void_p),
        ("row_sumsq", C.c_void_p),
        ("row_mean", C.c_void_p),
        ("row_rstd", C.c_void_p),
        ("eps", C.c_float),
        ("reserved", C.c_int32),
    ]


class GdpaQuantParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("in_is_fp32", C.c_int32),
        ("x", C.c_void_p),
        ("x8", C.c_void_p),
        ("scales", C.c_void_p),
        ("offsets", C.c_void_p),
        ("block_offsets", C.c_void_p),
        ("offsets_are_int64", C.c_int32),
        ("batch", C.c_int32),
        ("total", C.c_int64),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("scale_rows", C.c_int64),
    ]


class GdpaMxParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("x_is_fp32", C.c_int32),
        ("x", C.c_void_p),
        ("x8", C.c_void_p),
        ("sf", C.c_void_p),
        ("offsets", C.c_void_p),
        ("block_offsets", C.c_void_p),
        ("offsets_are_int64", C.c_int32),
        ("batch", C.c_int32),
        ("total", C.c_int64),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("scale_axis", C.c_int32),
        ("reserved", C.c_int32),
        ("sf_blocks", C.c_int64),
    ]


class GdpaNormBwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("mode", C.c_int32),
        ("rows", C.c_int64),
        ("n", C.c_int32),
        ("reserved", C.c_int32),
        ("dy", C.c_void_p),
        ("dy_add", C.c_void_p),
        ("x", C.c_void_p),
        ("dx", C.c_void_p),
        ("weight", C.c_void_p),
        ("row_mean", C.c_void_p),
        ("row_rstd", C.c_void_p),
        ("dweight", C.c_void_p),
        ("dbias", C.c_void_p),
    ]


class GdpaBwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("d_o", C.c_void_p),
        ("dq", C.c_void_p),
        ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("q_offsets", C.c_void_p),
        ("kv_offsets", C.c_void_p),
        ("offsets_are_int64", C.c_int32),
        ("batch", C.c_int32),
        ("total_q", C.c_int64),
        ("total_kv", C.c_int64),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("max_seq_len_q", C.c_int32),
        ("max_seq_len_kv", C.c_int32),
        ("activation", C.c_int32),
        ("qk_scale", C.c_float),
        ("schedule", C.c_void_p),
        ("dq_accum", C.c_void_p),
        ("status", C.c_void_p),
        ("timing_start_event", C.c_void_p),
        ("timing_stop_event", C.c_void_p),
        ("o", C.c_void_p),
        ("lse", C.c_void_p),
        ("dpsum", C.c_void_p),
        ("kv_heads", C.c_int32),
        ("window_plus_one", C.c_int32),
        ("q_strides", C.c_int64 * 2),
        ("k_strides", C.c_int64 * 2),
        ("v_strides", C.c_int64 * 2),
        ("dkv_accum", C.c_void_p),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ads_model_kernel_library_b200.build` "
            "(needs nvcc); this package has no other compute path"
        )
    lib = C.CDLL(LIB_PATH)
    lib.gdpa_schedule_bytes.restype = C.c_size_t
    lib.gdpa_schedule_bytes.argtypes = [C.c_int32, C.c_int64, C.c_int32, C.c_int32]
    lib.gdpa_build_schedule.restype = C.c_int
    lib.gdpa_build_schedule.argtypes = [C.POINTER(GdpaSchedParams), C.c_void_p]
    lib.gdpa_fwd.restype = C.c_int
    lib.gdpa_fwd.argtypes = [C.POINTER(GdpaFwdParams), C.c_void_p]
    lib.gdpa_fwd_noalloc.restype = C.c_int
    lib.gdpa_fwd_noalloc.argtypes = [C.POINTER(GdpaFwdParams), C.c_void_p]
    for fn in (lib.gdpa_layernorm_rows, lib.gdpa_rmsnorm_rows):
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(GdpaNormParams), C.c_void_p]
    lib.gdpa_quantize_fp8_blockwise.restype = C.c_int
    lib.gdpa_quantize_fp8_blockwise.argtypes = [C.POINTER(GdpaQuantParams), C.c_void_p]
    for fn in (lib.gdpa_quantize_mxfp8, lib.gdpa_dequantize_mxfp8):
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(GdpaMxParams), C.c_void_p]
    lib.gdpa_norm_rows_bwd.restype = C.c_int
    lib.gdpa_norm_rows_bwd.argtypes = [C.POINTER(GdpaNormBwdParams), C.c_void_p]
    lib.gdpa_fwd_fp8.restype = C.c_int
    lib.gdpa_fwd_fp8.argtypes = [C.POINTER(GdpaFwdParams), C.c_void_p]
    lib.gdpa_bwd_workspace_bytes.restype = C.c_size_t
    lib.gdpa_bwd_workspace_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32]
    lib.gdpa_bwd.restype = C.c_int
    lib.gdpa_bwd.argtypes = [C.POINTER(GdpaBwdParams), C.c_void_p]
    lib.gdpa_strerror.restype = C.c_char_p
    lib.gdpa_strerror.argtypes = [C.c_int]
    lib.gdpa_launch_count.restype = C.c_int64
    lib.gdpa_launch_count.argtypes = []
    lib.gdpa_debug_wait_probe.restype = C.c_int
    lib.gdpa_debug_wait_probe.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    lib.gdpa_debug_set_trace.restype = None
    lib.gdpa_debug_set_trace.argtypes = [C.c_void_p]
    lib.gdpa_version.restype = C.c_int32
    lib.gdpa_version.argtypes = []
    return lib


def __getattr__(name):
    # PEP 562: `_cabi.lib` is created by its first use and is an ordinary module attribute afterwards
    if name == "lib":
        globals()["lib"] = _load()
        return globals()["lib"]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def check(code: int, what: str) -> None:
    if code != GDPA_OK:
        handle = globals().get("lib") or __getattr__("lib")
        raise RuntimeError(f"{what}: {handle.gdpa_strerror(code).decode()} (code {code})")
