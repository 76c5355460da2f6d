"""CPU oracle for the RWKV7 generalized delta rule and the RWKV6 wkv operator.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module:
the product path is the CUDA library and it fails loudly when that library is
missing.  The oracle is used by the tests, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark, always as the
checker or the timed baseline and never as the thing being checked.

Parity pinning: the reference project ships no golden vectors for its native
operators.  The restatements here are pinned instead against outputs of the
reference's own ``native_keras_op.py`` and ``ops_rwkv_kernel.py`` files, loaded
unmodified through ``oracle.keras_shim`` and run on seeded inputs; those outputs
are committed as fixtures under ``tests/golden`` together with the script that
generated them.
"""
from .rwkv7_native import generalized_delta_rule, rwkv7_manual_backward  # noqa: F401
from .wkv6_native import RWKVKernelOperator, wkv6_manual_backward  # noqa: F401
