"""Decay inputs outside the benchmark distribution.

The chunked tensor-core kernels scale their operands around one reference point per 64-token chunk, which is
exact only while the decay summed over half a chunk stays within a limit; (batch, head) units beyond it are
marked on the device and recomputed by the float32 recurrence inside the same call.  These tests feed the
default (AUTO) path decays on both sides of the limit, including the distributions of the reference's own
smoke tests (``test_script/test_rwkv7_kernel.py:18``, ``test_script/test_rwkv6_kernel.py:18``: w ~ N(0,1)),
and compare with the CPU oracle.  Tolerance: relative L2 2e-2 for bfloat16 inputs, 1e-4 for float32.
"""
import pytest
import torch

import rwkv_ops_b200 as ro
from oracle import RWKVKernelOperator as OracleWkv6
from oracle import generalized_delta_rule as oracle_gdr
from rwkv_ops_b200 import _lib
from rwkv_ops_b200.workloads import rel_l2, rwkv7_inputs, wkv6_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _no_wait_ran_out():
    yield
    torch.cuda.synchronize()
    assert _lib.load().rwkvb200_device_status(1) == 0, "a bounded wait ran out inside a tensor-core kernel"


def _w_rwkv7(kind, shape, gen):
    """Raw decay inputs w (the operator applies g = -exp(w) per token and channel)."""
    n = torch.randn(shape, generator=gen)
    if kind == "mixed_in_range":      # per-channel |g| from 0 (the padding value) to 1.8, mixed inside a chunk
        g = 1.8 * torch.rand(shape, generator=gen)
        w = torch.log(g.clamp_min(1e-30))
        w[torch.rand(shape, generator=gen) < 0.1] = -1e9
        return w
    if kind == "edge":                # every channel close to the limit: 32 tokens sum to about 57
        return torch.log(1.75 + 0.05 * torch.rand(shape, generator=gen))
    if kind == "normal":              # w ~ N(0,1): |g| up to e^3 and more
        return n
    if kind == "fast":                # w ~ 1 + 0.3 N(0,1): |g| around e
        return 1.0 + 0.3 * n
    if kind == "one_unit_fast":       # only (batch 1, head 0) leaves the range
        w = -0.6 * torch.sigmoid(n)
        w[1, :, 0] = 1.0 + 0.3 * n[1, :, 0]
        return w
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["mixed_in_range", "edge", "normal", "fast", "one_unit_fast"])
@pytest.mark.parametrize("T", [96, 200])
def test_rwkv7_bf16_decay_range(kind, T):
    B, H = 2, 2
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=4100 + T, with_state=True, with_grads=True)
    d["w"] = _w_rwkv7(kind, d["w"].shape, torch.Generator().manual_seed(77)).to(torch.bfloat16)
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[ref[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref * d["d_out"].float()).sum() + (s_ref * d["d_state"]).sum()).backward()

    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    errs = {"o": rel_l2(o, o_ref), "s": rel_l2(s, s_ref), "dh0": rel_l2(h0.grad, h0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rwkvab"})
    assert all(torch.isfinite(t).all() for t in [o, s, h0.grad] + [g[n].grad for n in "rwkvab"])
    assert all(e < 2e-2 for e in errs.values()), (kind, {n: e for n, e in errs.items() if not e < 2e-2})


def test_rwkv7_out_of_range_units_equal_the_recurrence(monkeypatch):
    """A unit beyond the limit is recomputed by the very kernels of the recurrent path: its results carry
    the same bits, while the units inside the limit come from the tensor-core kernels."""
    B, T, H = 2, 130, 2
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=4300, with_grads=True)
    d["w"] = _w_rwkv7("one_unit_fast", d["w"].shape, torch.Generator().manual_seed(5)).to(torch.bfloat16)

    def run():
        g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
        o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"])
        torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
        return o, s, g

    o_a, s_a, g_a = run()
    monkeypatch.setenv("RWKV_OPS_B200_RWKV7_ALGO", "recurrent")
    o_r, s_r, g_r = run()
    assert torch.equal(o_a[1, :, 0], o_r[1, :, 0]) and torch.equal(s_a[1, 0], s_r[1, 0])
    for n in "rwkvab":
        assert torch.equal(g_a[n].grad[1, :, 0], g_r[n].grad[1, :, 0]), n
    assert not torch.equal(o_a[0], o_r[0])      # bfloat16-operand products differ in the last bits


def _w_wkv6(kind, shape, gen):
    n = torch.randn(shape, generator=gen)
    if kind == "normal":
        return n
    if kind == "fast":
        return 1.0 + 0.3 * n
    if kind == "one_row_fast":        # batch row 1 leaves the range, rows 0 and 2 stay inside
        w = -torch.exp(-0.5 + 0.5 * n)
        w[1] = 1.0 + 0.3 * n[1]
        return w
    if kind == "edge":                # every channel just inside the limit of the chunked path (32 x 1.35 < 45)
        return torch.log(1.3 + 0.05 * torch.rand(shape, generator=gen))
    if kind == "beyond_edge":         # and just outside it
        return torch.log(1.75 + 0.05 * torch.rand(shape, generator=gen))
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["normal", "fast", "one_row_fast", "edge", "beyond_edge"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [100, 193])
def test_wkv6_decay_range(kind, dtype, T):
    B, H = 3, 2
    d = wkv6_inputs(B, T, H, dtype=dtype, seed=4200 + T, n_state=2, with_grads=True)
    d["w"] = _w_wkv6(kind, d["w"].shape, torch.Generator().manual_seed(78)).to(dtype)
    d["state_map"] = torch.tensor([1, 0, 1], dtype=torch.int32)
    # float64 oracle: with decays this strong the float32 oracle's own gradient of w is off by several 1e-5
    ref = {n: d[n].double().clone().requires_grad_(True) for n in "rkvwu"}
    s0r = d["init_state"].double().clone().requires_grad_(True)
    y_ref, s_ref = OracleWkv6(64, T)(ref["r"], ref["k"], ref["v"], ref["w"], ref["u"], with_state=True,
                                     init_state=s0r, state_map=d["state_map"])
    ((y_ref * d["d_y"].double()).sum() + (s_ref * d["d_state"].double()).sum()).backward()

    g = {n: d[n].cuda().requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].cuda().requires_grad_(True)
    y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                              state_map=d["state_map"].cuda())
    ((y.float() * d["d_y"].cuda().float()).sum() + (s.float() * d["d_state"].cuda().float()).sum()).backward()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    errs = {"y": rel_l2(y, y_ref), "s": rel_l2(s, s_ref), "ds0": rel_l2(s0.grad, s0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rkvwu"})
    assert all(e < tol for e in errs.values()), (kind, {n: e for n, e in errs.items() if not e < tol})


def test_wkv6_inference_forward_out_of_range():
    """No gradients: the forward alone, without the chunk-boundary states of a training call."""
    B, T, H = 2, 150, 2
    d = wkv6_inputs(B, T, H, seed=4400)
    d["w"] = _w_wkv6("normal", d["w"].shape, torch.Generator().manual_seed(79))
    y_ref, s_ref = OracleWkv6(64, T)(d["r"], d["k"], d["v"], d["w"], d["u"], with_state=True)
    with torch.no_grad():
        y, s = ro.RWKV6_OP(64, T)(*[d[n].cuda() for n in "rkvwu"], with_state=True)
    assert rel_l2(y, y_ref) < 1e-4 and rel_l2(s, s_ref) < 1e-4


def test_rwkv7_out_of_range_units_with_head_first_layout_and_broadcast_state():
    """The recomputation of out-of-range units reads [B, H, T, 64] tensors and a broadcast initial state as
    the tensor-core kernels do: same results as the [B, T, H, 64] call on permuted tensors."""
    B, T, H = 2, 150, 3
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=4500, with_state=True, n_state=1, with_grads=True)
    d["w"] = _w_rwkv7("one_unit_fast", d["w"].shape, torch.Generator().manual_seed(6)).to(torch.bfloat16)

    def run(head_first):
        perm = (lambda t: t.permute(0, 2, 1, 3).contiguous()) if head_first else (lambda t: t)
        g = {n: perm(d[n].cuda()).requires_grad_(True) for n in "rwkvab"}
        h0 = d["initial_state"].cuda().requires_grad_(True)
        o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0, head_first=head_first)
        torch.autograd.backward([o, s], [perm(d["d_out"].cuda()), d["d_state"].cuda()])
        return perm(o), s, {n: perm(g[n].grad) for n in "rwkvab"}, h0.grad

    o0, s0, g0, dh0 = run(False)
    o1, s1, g1, dh1 = run(True)
    assert torch.equal(o0, o1) and torch.equal(s0, s1) and torch.equal(dh0, dh1)
    for n in "rwkvab":
        assert torch.equal(g0[n], g1[n]), n
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    o_ref, s_ref = oracle_gdr(*[ref[n] for n in "rwkvab"], initial_state=d["initial_state"])
    assert rel_l2(o0, o_ref) < 2e-2 and rel_l2(s0, s_ref) < 2e-2
