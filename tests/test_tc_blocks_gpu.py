"""The tcgen05 / TMA building blocks of the chunked path, one at a time on known data, through the
C ABI of the developer build of the library (``rwkvb200_tc_selftest``, ``include/rwkv_ops_b200_devtools.h``): 128-row MMA, paired 64-row MMAs with transposed (MN-major) operands,
TMA tiled load with zero fill past the end of the sequence, bulk store and bulk load."""
import pytest
import torch

from rwkv_ops_b200 import _lib

pytestmark = pytest.mark.gpu


def _mats(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(64, 64, generator=g).to(torch.bfloat16).cuda() for _ in range(4)]


def _status_clear(lib):
    assert lib.rwkvb200_device_status(1) == 0, "a bounded wait ran out in an earlier kernel"


def test_mma_128x128_kmajor():
    lib = _lib.load_dev()
    X, Y, Z, W = _mats(1)
    out = torch.zeros(128, 128, device="cuda")
    rc = lib.rwkvb200_tc_selftest(0, X.data_ptr(), Y.data_ptr(), Z.data_ptr(), W.data_ptr(), out.data_ptr(),
                                  None, 0, 0, 0, 0, 0, 0, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    ref = torch.cat([X, Y]).float() @ torch.cat([Z, W]).float().T
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3), (out - ref).abs().max()


def test_mma_64_pairs_with_transposed_operands():
    lib = _lib.load_dev()
    X, Y, Z, W = _mats(2)
    out = torch.zeros(128, 64, device="cuda")
    rc = lib.rwkvb200_tc_selftest(1, X.data_ptr(), Y.data_ptr(), Z.data_ptr(), W.data_ptr(), out.data_ptr(),
                                  None, 0, 0, 0, 0, 0, 0, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    r = torch.arange(64)
    lanes_lo = (r % 16) + 32 * (r // 16)
    lo = out[lanes_lo.cuda()]
    hi = out[(lanes_lo + 16).cuda()]
    ref_lo = X.float() @ Z.float()
    ref_hi = X.float().T @ W.float()
    assert torch.allclose(lo, ref_lo, rtol=1e-4, atol=1e-3), (lo - ref_lo).abs().max()
    assert torch.allclose(hi, ref_hi, rtol=1e-4, atol=1e-3), (hi - ref_hi).abs().max()


def test_mma_wide_and_long_transposed_operands():
    lib = _lib.load_dev()
    X, Y, Z, W = _mats(4)
    out = torch.zeros(128, 64, device="cuda")
    args = (X.data_ptr(), Y.data_ptr(), Z.data_ptr(), W.data_ptr(), out.data_ptr(), None, 0, 0, 0, 0, 0, 0, None)
    assert lib.rwkvb200_tc_selftest(3, *args, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    ref = torch.cat([X.float().T @ Z.float(), Y.float().T @ Z.float()])
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3), (out - ref).abs().max()
    out.zero_()
    assert lib.rwkvb200_tc_selftest(4, *args, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    r = torch.arange(64)
    lo = out[((r % 16) + 32 * (r // 16)).cuda()]
    ref = X.float().T @ Z.float() + Y.float().T @ W.float()
    assert torch.allclose(lo, ref, rtol=1e-4, atol=2e-3), (lo - ref).abs().max()


@pytest.mark.parametrize("t0,T", [(64, 192), (128, 150)])
def test_tma_tile_load_and_bulk_copies(t0, T):
    lib = _lib.load_dev()
    B, H, b, h = 2, 3, 1, 2
    g = torch.Generator().manual_seed(3)
    tok = torch.randn(B, T, H, 64, generator=g).to(torch.bfloat16).cuda()
    img = torch.zeros(2 * 4096, dtype=torch.bfloat16, device="cuda")
    rc = lib.rwkvb200_tc_selftest(2, None, None, None, None, None, tok.data_ptr(), B, T, H, b, t0, h,
                                  img.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    tile = torch.zeros(64, 64, dtype=torch.bfloat16)
    n = min(64, T - t0)
    tile[:n] = tok[b, t0:t0 + n, h].cpu()
    # expected shared-memory image: 16-byte chunk c of row r sits at chunk (c ^ (r & 7))
    exp = torch.zeros(64, 8, 8, dtype=torch.bfloat16)
    for r in range(64):
        for c in range(8):
            exp[r, c ^ (r & 7)] = tile[r, 8 * c:8 * c + 8]
    exp = exp.reshape(-1)
    assert torch.equal(img[:4096].cpu(), exp)
    assert torch.equal(img[4096:].cpu(), exp)


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns():
    """A bounded wait on a barrier that nothing ever completes (a thousand polls): the kernel gives up, winds
    down normally and the status word carries the code of the wait; the context stays usable."""
    lib = _lib.load_dev()
    _status_clear(lib)
    out = torch.zeros(4, device="cuda")
    rc = lib.rwkvb200_tc_selftest(5, None, None, None, None, out.data_ptr(), None, 0, 0, 0, 0, 0, 0, None,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.rwkvb200_device_status(1) == 105
    assert lib.rwkvb200_device_status(0) == 0      # cleared by the read above
    assert out[0].item() == 0.0
    X, Y, Z, W = _mats(9)                          # and the next kernel runs as usual
    o2 = torch.zeros(128, 128, device="cuda")
    assert lib.rwkvb200_tc_selftest(0, X.data_ptr(), Y.data_ptr(), Z.data_ptr(), W.data_ptr(), o2.data_ptr(),
                                    None, 0, 0, 0, 0, 0, 0, None, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    _status_clear(lib)
    ref = torch.cat([X, Y]).float() @ torch.cat([Z, W]).float().T
    assert torch.allclose(o2, ref, rtol=1e-4, atol=1e-3)
