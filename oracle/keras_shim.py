"""A minimal ``keras`` / ``keras.ops`` stand-in backed by torch (CPU).

TEST INFRASTRUCTURE ONLY.  The reference's two native operator files import
nothing but ``keras`` and ``keras.ops`` (``rwkv_ops/rwkv7_kernel/native_keras_op.py:1-2``,
``rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:1-2``) and keras is not installable
offline.  Registering this module as ``sys.modules["keras"]`` lets those files be
loaded *unmodified* with importlib so their outputs can be recorded as golden
vectors.  Only the ``keras.ops`` functions those two files call are provided.
"""
from __future__ import annotations

import importlib.util
import sys
import types

import torch

_DTYPES = {
    "float32": torch.float32,
    "float64": torch.float64,
    "bfloat16": torch.bfloat16,
    "float16": torch.float16,
    "int32": torch.int32,
    "int64": torch.int64,
}


def _dt(d):
    return _DTYPES[d] if isinstance(d, str) else d


def _cast(x, dtype):
    return x.to(_dt(dtype))


def _transpose(x, axes):
    return x.permute(*axes)


def _shape(x):
    return tuple(x.shape)


def _zeros(shape, dtype="float32"):
    return torch.zeros(tuple(shape), dtype=_dt(dtype))


def _reshape(x, shape):
    return x.reshape(tuple(shape))


def _broadcast_to(x, shape):
    return x.broadcast_to(tuple(shape))


def _slice_update(inputs, start_indices, updates):
    # keras semantics: functional update, returns a new tensor
    out = inputs.clone()
    idx = tuple(slice(int(s), int(s) + n) for s, n in zip(start_indices, updates.shape))
    out[idx] = updates
    return out


def _fori_loop(lower, upper, body_fun, init_val):
    val = init_val
    for i in range(int(lower), int(upper)):
        val = body_fun(i, val)
    return val


def _while_loop(cond, body, loop_vars, maximum_iterations=None):
    it = 0
    while cond(*loop_vars):
        if maximum_iterations is not None and it >= maximum_iterations:
            break
        loop_vars = tuple(body(*loop_vars))
        it += 1
    return loop_vars


def _take(x, indices, axis=None):
    if isinstance(indices, int):
        return x.select(axis, indices)
    return torch.index_select(x, axis, indices.to(torch.int64))


def _convert_to_tensor(x, dtype=None):
    return torch.as_tensor(x, dtype=_dt(dtype) if dtype is not None else None)


def install() -> types.ModuleType:
    """Register the stand-in as ``keras`` and ``keras.ops`` (idempotent)."""
    if "keras" in sys.modules and getattr(sys.modules["keras"], "_is_rwkv_oracle_shim", False):
        return sys.modules["keras"]
    keras = types.ModuleType("keras")
    ops = types.ModuleType("keras.ops")
    ops.cast = _cast
    ops.transpose = _transpose
    ops.shape = _shape
    ops.exp = torch.exp
    ops.zeros = _zeros
    ops.reshape = _reshape
    ops.broadcast_to = _broadcast_to
    ops.slice_update = _slice_update
    ops.fori_loop = _fori_loop
    ops.while_loop = _while_loop
    ops.take = _take
    ops.convert_to_tensor = _convert_to_tensor
    keras.ops = ops
    keras._is_rwkv_oracle_shim = True
    sys.modules["keras"] = keras
    sys.modules["keras.ops"] = ops
    return keras


def load_reference_module(path: str, name: str) -> types.ModuleType:
    """Load one reference source file, unmodified, under the stand-in keras."""
    install()
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
