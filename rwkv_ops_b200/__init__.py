"""rwkv_ops_b200: the RWKV7 generalized delta rule and the RWKV6 wkv operator on B200 (sm_100a).

Exports the same names as the reference package (``rwkv_ops/__init__.py:22-29``):
``generalized_delta_rule``, ``rwkv7_op``, ``RWKV7_USE_KERNEL``, ``get_generalized_delta_rule``,
``RWKV6_OP`` and ``get_rwkv6_kernel``.  The ``KERNEL_TYPE`` / ``KERAS_BACKEND`` environment
variables of the reference are not consulted: there is one implementation, hand-written CUDA
behind a C ABI, and it raises if its shared library is missing.  ``Rwkv7DecodeState`` (in-place
single-token decoding) ``generalized_delta_rule_varlen`` / ``wkv6_varlen`` (packed variable-length batches) and
``generalized_delta_rule_fused`` (the producers of w, a, b computed inside the operator) go beyond the
reference's working surface.
"""
from .rwkv7 import generalized_delta_rule, get_generalized_delta_rule
from .rwkv6 import RWKVKernelOperator, get_rwkv6_kernel
from .decode import Rwkv7DecodeState
from .varlen import PackedSequences, generalized_delta_rule_varlen, wkv6_varlen
from .fused import generalized_delta_rule_fused

__version__ = "0.1"

RWKV7_USE_KERNEL = True
rwkv7_op = generalized_delta_rule
RWKV6_OP = get_rwkv6_kernel()

__all__ = [
    "generalized_delta_rule",
    "rwkv7_op",
    "RWKV7_USE_KERNEL",
    "get_generalized_delta_rule",
    "RWKV6_OP",
    "get_rwkv6_kernel",
    "RWKVKernelOperator",
    "Rwkv7DecodeState",
    "generalized_delta_rule_varlen",
    "PackedSequences",
    "wkv6_varlen",
    "generalized_delta_rule_fused",
]
