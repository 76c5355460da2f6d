"""The workspace-free backward entry point (``rwkvb200_rwkv7_bwd_static``).

It exists for hosts that give an operator nothing but its input and output buffers and do not let
it call cudaMalloc (operator plugins of inference runtimes, servers with a fixed memory budget), so
its state checkpoints sit in a fixed array inside the library.  The test calls it through the C ABI
twice in a row, on different inputs, so that the second call runs on top of whatever the first left
in that array, and compares every output with the regular entry point, which uses a caller workspace.
The file is named so that pytest collects it last.
"""
import pytest
import torch

from rwkv_ops_b200 import _lib
from rwkv_ops_b200.workloads import rwkv7_inputs

pytestmark = pytest.mark.gpu


def _run_both(lib, B, T, H, dtype, seed, n_state):
    d = rwkv7_inputs(B, T, H, dtype=dtype, seed=seed, with_state=n_state > 0, n_state=n_state or None,
                     with_grads=True)
    x = {n: d[n].cuda().contiguous() for n in "rwkvab"}
    h0 = d["initial_state"].cuda() if n_state else None
    d_o, d_ht = d["d_out"].cuda(), d["d_state"].cuda()
    code = _lib.dtype_code(dtype)
    stream = torch.cuda.current_stream().cuda_stream

    def outputs():
        return [torch.empty_like(x["r"]) for _ in range(6)] + [torch.empty(B, H, 64, 64, device="cuda")]

    ref = outputs()
    nws = lib.rwkvb200_rwkv7_bwd_workspace_bytes(B, T, H, 64, code, _lib.ALGO_RECURRENT)
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda")
    rc = lib.rwkvb200_rwkv7_bwd(*[x[n].data_ptr() for n in "rwkvab"], _lib.ptr(h0), n_state, d_o.data_ptr(),
                                d_ht.data_ptr(), *[t.data_ptr() for t in ref], ws.data_ptr(), nws,
                                B, T, H, 64, code, 0, _lib.ALGO_RECURRENT, stream)
    assert rc == 0, _lib.strerror(rc)
    got = outputs()
    before = torch.cuda.memory_allocated()
    rc = lib.rwkvb200_rwkv7_bwd_static(*[x[n].data_ptr() for n in "rwkvab"], _lib.ptr(h0), n_state, d_o.data_ptr(),
                                       d_ht.data_ptr(), *[t.data_ptr() for t in got], B, T, H, 64, code, 0, stream)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return ref, got


def test_static_backward_matches_workspace_backward_twice_in_a_row():
    assert torch.cuda.is_available()
    lib = _lib.load()
    assert lib.rwkvb200_rwkv7_bwd_static_capacity_bytes() == 32 << 20
    # first call, then a second one with other shapes and values on top of the first call's leftovers
    for (B, T, H, dtype, seed, n_state) in [(2, 100, 3, torch.float32, 901, 2), (3, 37, 2, torch.bfloat16, 902, 0)]:
        ref, got = _run_both(lib, B, T, H, dtype, seed, n_state)
        for name, a, b in zip(["dr", "dw", "dk", "dv", "da", "db", "dh0"], ref, got):
            # same kernels, same arithmetic: only the place of the checkpoints differs
            assert torch.equal(a, b), name


def test_static_backward_rejects_sizes_beyond_its_array():
    lib = _lib.load()
    A = 0x1000   # never dereferenced: the size check fails first
    # 64 * 64 units * 128 checkpoints * 16 KiB = 8 GiB of checkpoints
    rc = lib.rwkvb200_rwkv7_bwd_static(*([A] * 6), None, 0, A, None, *([A] * 6), None, 64, 1024, 64, 64, 0, 0, None)
    assert rc == -9 and "capacity" in _lib.strerror(rc)
