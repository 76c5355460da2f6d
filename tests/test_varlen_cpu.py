"""Host-side logic of the packed variable-length entry: cu_seqlens handling (no GPU needed)."""
import pytest
import torch

from rwkv_ops_b200.varlen import _seq_arrays, _token_args, generalized_delta_rule_varlen
from rwkv_ops_b200 import _lib


def test_seq_arrays_from_list_and_tensor():
    for cu_in in ([0, 3, 10, 11], torch.tensor([0, 3, 10, 11]), torch.tensor([0, 3, 10, 11], dtype=torch.int32)):
        cu, start, lens, max_len = _seq_arrays(cu_in, 11, "cpu")
        assert cu.tolist() == [0, 3, 10, 11]
        assert start.tolist() == [0, 3, 10] and start.dtype == torch.int32
        assert lens.tolist() == [3, 7, 1] and lens.dtype == torch.int32
        assert max_len == 7


@pytest.mark.parametrize("cu,total", [
    ([0], 0),               # no sequence
    ([1, 5], 5),            # does not start at 0
    ([0, 4], 5),            # does not cover every token
    ([0, 3, 3, 5], 5),      # an empty sequence
    ([0, 4, 2, 5], 5),      # not increasing
])
def test_seq_arrays_rejects(cu, total):
    with pytest.raises(ValueError):
        _seq_arrays(cu, total, "cpu")


def test_varlen_needs_cuda_tensors():
    x = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(_lib.RwkvB200Error):
        generalized_delta_rule_varlen(x, x, x, x, x, x, [0, 4])


def test_token_tensors_are_cast_to_the_dtype_of_r():
    """Mixed dtypes (w in float32 beside bfloat16 r) must not reach the kernels, which read one element type."""
    r = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    w = torch.full((1, 4, 2, 64), -0.5, dtype=torch.float32)
    out = _token_args(r, w, r, r, r.transpose(1, 2).contiguous().transpose(1, 2), r)
    assert all(t.dtype == torch.bfloat16 and t.is_contiguous() for t in out)
    assert torch.equal(out[1], w.to(torch.bfloat16))
