"""Activation names and integer ids, as the reference library enumerates them
(gdpa/triton/math.py:43-55, ids by enumeration order :77-78), plus ``softmax``."""
from __future__ import annotations

from enum import Enum
from typing import Optional


class Activation(str, Enum):
    Raw = "raw"
    GeLU = "gelu"
    GeLUApprox = "gelu_approx"
    FastGeLU = "fast_gelu"
    LeakyReLU = "leaky_relu"
    ReLU = "relu"
    FastGeLUBF16 = "fast_gelu_bf16"
    SiLu = "silu"
    FastSiLu = "fast_silu"
    HardSwish = "hardswish"
    ReLUSquare = "relu_square"
    FastGeLUTaylorApprox = "fast_gelu_taylor_approx"


activation_to_int = {act: i for i, act in enumerate(Activation)}
int_to_activation = {i: act for act, i in activation_to_int.items()}

SOFTMAX = "softmax"
SOFTMAX_ID = 100


def activation_string_to_int(s: str) -> Optional[int]:
    """Id of a reference activation name; ValueError for an unknown one
    (gdpa/triton/math.py:81-85).  ``softmax`` maps to this library's id 100."""
    if s == SOFTMAX:
        return SOFTMAX_ID
    if s not in Activation._value2member_map_:
        raise ValueError(f"Unsupported activation function: {s}")
    return activation_to_int.get(Activation(s))
