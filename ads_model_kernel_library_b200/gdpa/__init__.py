"""GDPA operator package: drop-in for the reference's ``gdpa`` entry point."""
from .host_pipeline import forward_backward_host  # noqa: F401
from .math import Activation, activation_string_to_int, activation_to_int, int_to_activation  # noqa: F401
from .megakernel import gdpa_megakernel, layernorm_rows, rmsnorm_rows, tlx_gdpa_megakernel  # noqa: F401
from .mxfp8 import dequantize_mxfp8, generalized_dot_product_attention_mxfp8, quantize_varlen_mxfp8_sf_only  # noqa: F401
from .ops import (  # noqa: F401
    expect_contiguous,
    generalized_dot_product_attention,
    generalized_dot_product_attention_fp8,
    kernel_status,
    kernel_timing,
    quantize_fp8_blockwise,
    set_offset_validation,
)
from .sharding import gather_rows, max_over_ranks, plan_token_balanced_shards, shard_inputs, shard_jagged  # noqa: F401
from .workloads import WORKLOADS, make_workload, useful_flops  # noqa: F401
