"""ctypes binding of librwkv_ops_b200.so (the C ABI declared in include/rwkv_ops_b200.h).

There is no fallback: if the shared library is missing or an entry point returns an
error code, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_size_t, c_void_p, c_char_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# RWKV_OPS_B200_LIBRARY selects another build of the library (e.g. the developer build, to profile with its
# phase stamps); default: the library built in-tree next to this file
LIB_PATH = os.environ.get("RWKV_OPS_B200_LIBRARY") or os.path.join(_PKG, "librwkv_ops_b200.so")
DEV_LIB_PATH = os.path.join(_PKG, "librwkv_ops_b200_dev.so")

F32, BF16, F16 = 0, 1, 2
ALGO_AUTO, ALGO_RECURRENT, ALGO_CHUNKED = 0, 1, 2
ALGO_KEEP = 0x100
PHASE_PREPARE, PHASE_SCAN, PHASE_FINISH = 0x1000, 0x2000, 0x4000
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

# name -> (restype, argtypes); mirrors include/rwkv_ops_b200.h one to one
_P, _I, _Z = c_void_p, c_int, c_size_t
SIGNATURES = {
    "rwkvb200_abi_version": (c_int, []),
    "rwkvb200_strerror": (c_char_p, [_I]),
    "rwkvb200_last_cuda_error": (c_char_p, []),
    "rwkvb200_rwkv7_step": (c_int, [_P] * 6 + [_P, _I, _P, _P, _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_decode_step": (c_int, [_P] * 6 + [_P, _I, _P, _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_fused_fwd": (c_int, [_P] * 6 + [_P, _I, _P, _P, _P, c_size_t, _I, _I, _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_fused_bwd": (c_int, [_P] * 6 + [_P, _I, _P, _P] + [_P] * 7 +
                                 [_P, c_size_t, _I, _I, _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_varlen_workspace_bytes": (c_size_t, [_I] * 5),
    "rwkvb200_rwkv7_fwd_varlen": (c_int, [_P] * 6 + [_P, _P, _I, _I, _I, _P, _I, _P, _P, _P, c_size_t,
                                                      _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_bwd_varlen": (c_int, [_P] * 6 + [_P, _P, _I, _I, _I, _P, _I, _P, _P] + [_P] * 7 +
                                  [_P, c_size_t, _I, _I, _I, _I, _P]),
    "rwkvb200_rwkv7_fwd_workspace_bytes": (c_size_t, [_I] * 6),
    "rwkvb200_rwkv7_fwd": (c_int, [_P] * 6 + [_P, _I, _P, _P, _P, _Z] + [_I] * 7 + [_P]),
    "rwkvb200_rwkv7_bwd_workspace_bytes": (c_size_t, [_I] * 6),
    "rwkvb200_rwkv7_bwd": (c_int, [_P] * 6 + [_P, _I, _P, _P] + [_P] * 7 + [_P, _Z] + [_I] * 7 + [_P]),
    "rwkvb200_rwkv7_bwd_static_capacity_bytes": (c_size_t, []),
    "rwkvb200_rwkv7_bwd_static": (c_int, [_P] * 6 + [_P, _I, _P, _P] + [_P] * 7 + [_I] * 6 + [_P]),
    "rwkvb200_wkv6_fwd_workspace_bytes": (c_size_t, [_I] * 6),
    "rwkvb200_wkv6_fwd": (c_int, [_P] * 5 + [_P, _I, _P, _P, _P, _P, _Z] + [_I] * 6 + [_P]),
    "rwkvb200_wkv6_bwd_workspace_bytes": (c_size_t, [_I] * 6),
    "rwkvb200_wkv6_bwd": (c_int, [_P] * 5 + [_P, _I, _P, _P, _P] + [_P] * 6 + [_P, _Z] + [_I] * 6 + [_P]),
    "rwkvb200_wkv6_varlen_workspace_bytes": (c_size_t, [_I] * 6),
    "rwkvb200_wkv6_fwd_varlen": (c_int, [_P] * 5 + [_P, _P, _I, _I, _I, _P, _I, _P, _P, _P, _P, _Z] + [_I] * 4 + [_P]),
    "rwkvb200_wkv6_bwd_varlen": (c_int, [_P] * 5 + [_P, _P, _I, _I, _I, _P, _I, _P, _P, _P] + [_P] * 6 + [_P, _Z] +
                                 [_I] * 4 + [_P]),
    "rwkvb200_device_status": (c_int, [_I]),
    "rwkvb200_profile_enable": (None, [_I]),
    "rwkvb200_profile_reset": (None, []),
    "rwkvb200_profile_count": (c_int, []),
    "rwkvb200_profile_get": (c_int, [_I, c_char_p, _I, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(c_int)]),
}

# the developer build adds these (include/rwkv_ops_b200_devtools.h)
DEV_SIGNATURES = {
    "rwkvb200_debug_stamps": (None, [_P]),
    "rwkvb200_tc_selftest": (c_int, [_I] + [_P] * 6 + [_I] * 6 + [_P, _P]),
}

_lib = None
_dev_lib = None


class RwkvB200Error(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RwkvB200Error(
            f"{LIB_PATH} not found. Build it with `python -m rwkv_ops_b200.build` (needs nvcc); "
            "rwkv_ops_b200 has no CPU or eager fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    got = lib.rwkvb200_abi_version()
    if got != 1:
        raise RwkvB200Error(f"ABI version mismatch: library {got}, binding 1")
    _lib = lib
    return lib


def load_dev() -> ctypes.CDLL:
    """The developer build of the library (``python -m rwkv_ops_b200.build --dev``): every product entry point
    plus the self-test and phase-stamp entry points.  Used by the unit tests of the tensor-core building blocks
    only; it is a separate library with its own device state."""
    global _dev_lib
    if _dev_lib is not None:
        return _dev_lib
    if not os.path.exists(DEV_LIB_PATH):
        raise RwkvB200Error(f"{DEV_LIB_PATH} not found. Build it with `python -m rwkv_ops_b200.build --dev`.")
    lib = ctypes.CDLL(DEV_LIB_PATH)
    for name, (res, args) in {**SIGNATURES, **DEV_SIGNATURES}.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _dev_lib = lib
    return lib


def check_status(what: str) -> None:
    """With ``RWKV_OPS_B200_CHECK_STATUS=1``: synchronise and raise if a bounded wait inside a tensor-core
    kernel ran out during ``what`` (the kernel then wound down and its results are not valid).  Off by
    default, because it synchronises the device after every operator call."""
    if os.environ.get("RWKV_OPS_B200_CHECK_STATUS", "0") not in ("", "0"):
        code = load().rwkvb200_device_status(1)
        if code != 0:
            raise RwkvB200Error(f"{what}: a bounded wait inside a tensor-core kernel ran out (code {code}); "
                                "the results of this call are not valid")


def _a256(x: int) -> int:
    return (x + 255) & ~255


def rwkv7_kept_bytes(n_seq: int, max_len: int, H: int) -> int:
    """Size of the tile store a training forward of the chunked RWKV7 path hands to its backward: the value of
    ``rwkvb200_rwkv7_fwd_workspace_bytes(..., ALGO_KEEP)`` without calling into the library (the shape
    functions of the custom ops must run without a device)."""
    n = n_seq * H * ((max_len + 63) // 64)
    return _a256(n * 18 * 8192) + _a256(n * 128 * 4) + _a256(n_seq * H * 4) + 1024


def wkv6_kept_bytes(B: int, T: int, H: int) -> int:
    """Likewise for ``rwkvb200_wkv6_fwd_workspace_bytes(..., ALGO_KEEP)``."""
    nt = (T + 63) // 64
    return (_a256(B * H * (nt + 1) * 64 * 64 * 4) + _a256(B * H * 2 * 64 * 4) + _a256(B * H * 4 * 64 * 4)
            + _a256(B * H * 4) + _a256(B * H * 64 * 64 * 4) + _a256((B * H + 1) * 4))


def strerror(code: int) -> str:
    return load().rwkvb200_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code == 0:
        return
    msg = f"{what}: {strerror(code)} (code {code})"
    if code == -7:
        msg += f": {load().rwkvb200_last_cuda_error().decode()}"
    if code in (-1, -2, -3, -4, -6, -8, -9):
        raise ValueError(msg)
    raise RwkvB200Error(msg)


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported token dtype {dt}; use float32, bfloat16 or float16") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RwkvB200Error(
                "rwkv_ops_b200 operators run on CUDA tensors only (got a tensor on "
                f"{t.device}); there is no CPU fallback."
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("all tensors must be on the same device")
    return dev


def profile(on: bool) -> None:
    """Switch per-kernel event timing on (after clearing old records) or off."""
    lib = load()
    if on:
        lib.rwkvb200_profile_reset()
    lib.rwkvb200_profile_enable(int(on))


def profile_results() -> dict:
    """{kernel name: (total_ms, launches)} of everything launched since ``profile(True)``."""
    lib = load()
    out = {}
    for i in range(lib.rwkvb200_profile_count()):
        name = ctypes.create_string_buffer(96)
        ms, n = ctypes.c_float(), c_int()
        check(lib.rwkvb200_profile_get(i, name, 96, ctypes.byref(ms), ctypes.byref(n)), "profile_get")
        out[name.value.decode()] = (ms.value, n.value)
    return out
