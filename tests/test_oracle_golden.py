"""The CPU oracle against the golden vectors recorded from the reference's native operators."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import generalized_delta_rule, rwkv7_manual_backward, RWKVKernelOperator, wkv6_manual_backward
from rwkv_ops_b200.workloads import rel_l2

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
R7 = sorted(glob.glob(os.path.join(GOLDEN, "rwkv7_*.npz")))
R6 = sorted(glob.glob(os.path.join(GOLDEN, "wkv6_*.npz")))


def _t(z, key, dtype=None):
    if key not in z:
        return None
    t = torch.from_numpy(z[key])
    return t.to(dtype) if dtype is not None else t


def test_fixtures_present():
    assert len(R7) >= 5 and len(R6) >= 4


@pytest.mark.parametrize("path", R7, ids=[os.path.basename(p) for p in R7])
def test_rwkv7_oracle_matches_reference(path):
    z = np.load(path)
    dt = getattr(torch, str(z["dtype"]))
    ins = {n: _t(z, f"in_{n}", dt).requires_grad_(True) for n in "rwkvab"}
    h0 = _t(z, "in_initial_state")
    if h0 is not None:
        h0.requires_grad_(True)
    o, s = generalized_delta_rule(ins["r"], ins["w"], ins["k"], ins["v"], ins["a"], ins["b"], initial_state=h0)
    assert o.dtype == dt and s.dtype == torch.float32
    # same float32 arithmetic in the same order: differences are rounding noise only
    assert rel_l2(o, _t(z, "o")) < 2e-6
    assert rel_l2(s, _t(z, "final_state")) < 2e-6
    loss = (o.float() * _t(z, "d_out")).sum() + (s * _t(z, "d_state")).sum()
    loss.backward()
    for n in "rwkvab":
        tol = 2e-5 if dt == torch.float32 else 1e-2  # bf16 leaves round their gradients to bf16
        assert rel_l2(ins[n].grad, _t(z, f"grad_{n}")) < tol, n
    if h0 is not None:
        assert rel_l2(h0.grad, _t(z, "grad_initial_state")) < 2e-5


@pytest.mark.parametrize("path", R7, ids=[os.path.basename(p) for p in R7])
def test_rwkv7_manual_backward_matches_reference_autograd(path):
    z = np.load(path)
    if str(z["dtype"]) != "float32":
        pytest.skip("bf16 fixture gradients are rounded to bf16")
    ins = [_t(z, f"in_{n}") for n in "rwkvab"]
    h0 = _t(z, "in_initial_state")
    g = rwkv7_manual_backward(*ins, h0, _t(z, "d_out"), _t(z, "d_state"))
    for n, gn in zip("rwkvab", g[:6]):
        assert rel_l2(gn, _t(z, f"grad_{n}")) < 2e-5, n
    if h0 is not None:
        gs = g[6]
        if h0.shape[0] == 1:
            gs = gs.sum(0, keepdim=True)
        assert rel_l2(gs, _t(z, "grad_initial_state")) < 2e-5


@pytest.mark.parametrize("path", R6, ids=[os.path.basename(p) for p in R6])
def test_wkv6_oracle_matches_reference(path):
    z = np.load(path)
    ins = {n: _t(z, f"in_{n}").requires_grad_(True) for n in "rkvwu"}
    s0 = _t(z, "in_init_state")
    if s0 is not None:
        s0.requires_grad_(True)
    smap = _t(z, "in_state_map")
    with_state = "final_state" in z
    B, T, C = ins["r"].shape
    op = RWKVKernelOperator(64, T)
    y, s = op(ins["r"], ins["k"], ins["v"], ins["w"], ins["u"], with_state=with_state, init_state=s0, state_map=smap)
    assert rel_l2(y, _t(z, "y")) < 2e-6
    loss = (y * _t(z, "d_y")).sum()
    if with_state:
        assert rel_l2(s, _t(z, "final_state")) < 2e-6
        loss = loss + (s * _t(z, "d_state")).sum()
    else:
        assert s is None
    loss.backward()
    for n in "rkvwu":
        assert rel_l2(ins[n].grad, _t(z, f"grad_{n}")) < 2e-5, n
    if s0 is not None:
        assert rel_l2(s0.grad, _t(z, "grad_init_state")) < 2e-5
    # hand-derived reverse recurrence agrees with the reference's autograd gradients
    n_state = 0 if s0 is None else s0.shape[0]
    if smap is None and s0 is not None:
        smap = torch.zeros(B, dtype=torch.int64) if n_state == 1 else torch.arange(B)
    s0b = None if s0 is None else s0.detach().index_select(0, smap.long())
    g = wkv6_manual_backward(*[ins[n].detach() for n in "rkvwu"], s0b, _t(z, "d_y"),
                             _t(z, "d_state") if with_state else None, 64)
    for n, gn in zip("rkvwu", g[:5]):
        assert rel_l2(gn.reshape(z[f"grad_{n}"].shape), _t(z, f"grad_{n}")) < 2e-5, n
    if s0 is not None:
        ds0 = torch.zeros(n_state, *g[5].shape[1:], dtype=g[5].dtype).index_add_(0, smap.long(), g[5])
        assert rel_l2(ds0, _t(z, "grad_init_state")) < 2e-5


def test_rwkv7_oracle_head_first_is_a_permutation():
    z = np.load(os.path.join(GOLDEN, "rwkv7_t19_nostate.npz"))
    ins = [_t(z, f"in_{n}") for n in "rwkvab"]
    o_ref = _t(z, "o")
    o_hf, s_hf = generalized_delta_rule(*[x.permute(0, 2, 1, 3).contiguous() for x in ins], head_first=True)
    assert o_hf.shape == (o_ref.shape[0], o_ref.shape[2], o_ref.shape[1], o_ref.shape[3])
    assert rel_l2(o_hf.permute(0, 2, 1, 3), o_ref) < 2e-6
    o_only = generalized_delta_rule(*ins, output_final_state=False)
    assert torch.is_tensor(o_only)


def test_wkv6_oracle_state_map_errors():
    op = RWKVKernelOperator(64, 8)
    x = torch.zeros(3, 4, 64)
    with pytest.raises(ValueError):
        op(x, x, x, x, torch.zeros(64), with_state=True, init_state=torch.zeros(2, 1, 64, 64))
    with pytest.raises(AssertionError):
        op(x, x, x, x, torch.zeros(64), with_state=True, init_state=torch.zeros(2, 1, 64, 64), state_map=[0, 1, 2])
