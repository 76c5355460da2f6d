"""Host-side checks of the C-ABI library that need no GPU: it loads, exports every declared
symbol, and rejects bad arguments with the documented codes before anything is launched."""
import ctypes
import os
import re

import pytest

from rwkv_ops_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rwkv_ops_b200.h")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from rwkv_ops_b200.build import build
        build()
    return _lib.load()


def _declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rwkvb200_\w+)\s*\(", src)))


def test_header_and_binding_agree(lib):
    declared = _declared_symbols()
    assert len(declared) >= 10
    assert set(declared) == set(_lib.SIGNATURES), "include/rwkv_ops_b200.h and _lib.SIGNATURES differ"
    for name in declared:
        assert hasattr(lib, name), f"library does not export {name}"


def test_abi_version_and_strerror(lib):
    assert lib.rwkvb200_abi_version() == 1
    assert _lib.strerror(0) == "ok"
    for code in range(-9, 0):
        assert _lib.strerror(code) != "unknown error code"
    assert _lib.strerror(-99) == "unknown error code"


def test_argument_validation_without_launch(lib):
    A = 0x1000  # a fake, 16-byte aligned address; never dereferenced because validation fails first
    six = [A] * 6
    # bad sizes
    assert lib.rwkvb200_rwkv7_step(*six, A, 1, A, A, 0, 4, 64, 0, None) == -1
    # unsupported head size
    assert lib.rwkvb200_rwkv7_step(*six, A, 1, A, A, 2, 4, 32, 0, None) == -6
    # bad dtype
    assert lib.rwkvb200_rwkv7_step(*six, A, 1, A, A, 2, 4, 64, 7, None) == -2
    # null pointer
    assert lib.rwkvb200_rwkv7_step(None, *six[1:], A, 1, A, A, 2, 4, 64, 0, None) == -4
    # misaligned pointer
    assert lib.rwkvb200_rwkv7_step(A + 4, *six[1:], A, 1, A, A, 2, 4, 64, 0, None) == -3
    # n_state must be 0, 1 or B
    assert lib.rwkvb200_rwkv7_fwd(*six, A, 3, A, A, None, 0, 2, 8, 4, 64, 0, 0, 1, None) == -1
    # workspace too small for the backward
    need = lib.rwkvb200_rwkv7_bwd_workspace_bytes(2, 8, 4, 64, 0, 1)
    assert need >= 2 * 4 * 64 * 64 * 4
    assert lib.rwkvb200_rwkv7_bwd(*six, None, 0, A, None, *([A] * 6), None, A, need - 1,
                                  2, 8, 4, 64, 0, 0, 1, None) == -5
    # wkv6: several initial states and no state_map, n_state != B
    assert lib.rwkvb200_wkv6_fwd(*([A] * 5), A, 3, None, A, None, None, 0, 2, 8, 4, 64, 0, 0, None) == -8
    assert lib.rwkvb200_wkv6_bwd_workspace_bytes(2, 8, 4, 64, 0, 1) > 0
    # wkv6 head sizes: 32 and 128 through the recurrence (checkpoints every 8 tokens + one du row per CTA),
    # anything else and the chunked path at a head size other than 64 are unsupported
    assert lib.rwkvb200_wkv6_bwd_workspace_bytes(2, 8, 4, 32, 0, 1) == 2 * 4 * 32 * 32 * 4 + 2 * 4 * 2 * 32 * 4
    assert lib.rwkvb200_wkv6_bwd_workspace_bytes(2, 8, 4, 128, 0, 0) == 2 * 4 * 128 * 128 * 4 + 2 * 4 * 8 * 128 * 4
    assert lib.rwkvb200_wkv6_bwd_workspace_bytes(2, 8, 4, 48, 0, 1) == 0
    assert lib.rwkvb200_wkv6_bwd_workspace_bytes(2, 8, 4, 128, 0, 2) == 0
    assert lib.rwkvb200_wkv6_fwd(*([A] * 5), None, 0, None, A, None, None, 0, 2, 8, 4, 48, 0, 0, None) == -6
    assert lib.rwkvb200_wkv6_fwd(*([A] * 5), None, 0, None, A, None, None, 0, 2, 8, 4, 128, 0, 2, None) == -6


def test_python_layer_refuses_cpu_tensors():
    import torch
    import rwkv_ops_b200 as ro

    x = torch.zeros(1, 4, 2, 64)
    with pytest.raises(_lib.RwkvB200Error):
        ro.generalized_delta_rule(x, x, x, x, x, x)
    op = ro.RWKV6_OP(64, 16)
    y = torch.zeros(1, 4, 128)
    with pytest.raises(_lib.RwkvB200Error):
        op(y, y, y, y, torch.zeros(128))


def test_reference_api_surface():
    import inspect
    import rwkv_ops_b200 as ro

    sig = inspect.signature(ro.generalized_delta_rule)
    assert list(sig.parameters) == ["r", "w", "k", "v", "a", "b", "initial_state", "output_final_state", "head_first"]
    assert sig.parameters["output_final_state"].default is True and sig.parameters["head_first"].default is False
    fn, use_kernel = ro.get_generalized_delta_rule(64)
    assert fn is ro.generalized_delta_rule and use_kernel is True and ro.RWKV7_USE_KERNEL is True
    assert ro.rwkv7_op is ro.generalized_delta_rule
    sig6 = inspect.signature(ro.RWKV6_OP.__call__)
    assert list(sig6.parameters) == ["self", "r", "k", "v", "w", "u", "with_state", "init_state", "state_map"]
    assert list(inspect.signature(ro.RWKV6_OP.__init__).parameters) == ["self", "head_size", "max_sequence_length", "ops_loop"]
    assert ro.get_rwkv6_kernel("cuda") is ro.RWKV6_OP


def test_python_mirrors_of_the_kept_sizes_match_the_library(lib):
    """The shape functions of the custom ops (register_fake) size the tile store a training forward returns
    without calling the library; they must agree with it."""
    keep = _lib.ALGO_KEEP
    for (B, T, H) in [(1, 1, 1), (2, 64, 3), (3, 65, 2), (8, 4096, 32), (5, 1000, 7)]:
        assert _lib.rwkv7_kept_bytes(B, T, H) == lib.rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, 64, _lib.BF16, keep)
        assert _lib.rwkv7_kept_bytes(B, T, H) == lib.rwkvb200_rwkv7_varlen_workspace_bytes(B, T, H, 64, 1)
        assert _lib.wkv6_kept_bytes(B, T, H) == lib.rwkvb200_wkv6_fwd_workspace_bytes(B, T, H, 64, _lib.F32, keep)
        assert _lib.wkv6_kept_bytes(B, T, H) == lib.rwkvb200_wkv6_bwd_workspace_bytes(B, T, H, 64, _lib.F32, 0)
