"""GPU parity of the RWKV6 wkv operator against the CPU oracle and the golden vectors recorded
from the reference's native operator.  Tolerance: relative L2 1e-4 for float32, 2e-2 for bfloat16."""
import glob
import os

import numpy as np
import pytest
import torch

import rwkv_ops_b200 as ro
from oracle import RWKVKernelOperator as OracleOp, wkv6_manual_backward
from rwkv_ops_b200.workloads import wkv6_inputs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["auto", "recurrent"])
def _algo(request, monkeypatch):
    """Every test runs on the chunked tensor-core path (auto) and on the float32 recurrence."""
    monkeypatch.setenv("RWKV_OPS_B200_WKV6_ALGO", request.param)
    yield request.param
    torch.cuda.synchronize()
    from rwkv_ops_b200 import _lib
    assert _lib.load().rwkvb200_device_status(1) == 0, "a bounded wait ran out inside a tensor-core kernel"

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
R6 = sorted(glob.glob(os.path.join(GOLDEN, "wkv6_*.npz")))


@pytest.mark.parametrize("path", R6, ids=[os.path.basename(p)[:-4] for p in R6])
def test_golden_forward_backward(path):
    z = np.load(path)
    ins = {n: torch.from_numpy(z[f"in_{n}"]).cuda().requires_grad_(True) for n in "rkvwu"}
    s0 = torch.from_numpy(z["in_init_state"]).cuda().requires_grad_(True) if "in_init_state" in z else None
    smap = torch.from_numpy(z["in_state_map"]).cuda() if "in_state_map" in z else None
    with_state = "final_state" in z
    T = ins["r"].shape[1]
    y, s = ro.RWKV6_OP(64, T)(ins["r"], ins["k"], ins["v"], ins["w"], ins["u"], with_state=with_state,
                              init_state=s0, state_map=smap)
    assert rel_l2(y, torch.from_numpy(z["y"])) < 1e-4
    loss = (y * torch.from_numpy(z["d_y"]).cuda()).sum()
    if with_state:
        assert rel_l2(s, torch.from_numpy(z["final_state"])) < 1e-4
        loss = loss + (s * torch.from_numpy(z["d_state"]).cuda()).sum()
    else:
        assert s is None
    loss.backward()
    for n in "rkvwu":
        assert ins[n].grad.shape == ins[n].shape
        assert rel_l2(ins[n].grad, torch.from_numpy(z[f"grad_{n}"])) < 1e-4, n
    if s0 is not None:
        assert rel_l2(s0.grad, torch.from_numpy(z["grad_init_state"])) < 1e-4


@pytest.mark.parametrize("T", [1, 2, 7, 8, 9, 31, 64, 100])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_lengths_vs_oracle(T, dtype):
    B, H = 3, 2
    d = wkv6_inputs(B, T, H, dtype=dtype, seed=600 + T, n_state=2, with_grads=True)
    d["state_map"] = torch.tensor([1, 0, 1], dtype=torch.int32)   # a repeated table row
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rkvwu"}
    s0r = d["init_state"].float().clone().requires_grad_(True)
    y_ref, s_ref = OracleOp(64, T)(ref["r"], ref["k"], ref["v"], ref["w"], ref["u"], with_state=True,
                                   init_state=s0r, state_map=d["state_map"])
    ((y_ref * d["d_y"].float()).sum() + (s_ref * d["d_state"].float()).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].cuda().requires_grad_(True)
    y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                              state_map=d["state_map"].cuda())
    assert y.dtype == dtype and s.dtype == dtype
    ((y.float() * d["d_y"].cuda().float()).sum() + (s.float() * d["d_state"].cuda().float()).sum()).backward()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel_l2(y, y_ref) < tol and rel_l2(s, s_ref) < tol
    for n in "rkvwu":
        assert rel_l2(g[n].grad, ref[n].grad) < tol, n
    assert rel_l2(s0.grad, s0r.grad) < tol


@pytest.mark.parametrize("N", [32, 128])
@pytest.mark.parametrize("T", [1, 9, 70])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_head_sizes_32_and_128(N, T, dtype, tol):
    """The operator's constructor takes the head size (rwkv6_kernel/__init__.py:37-50): 32 and 128 against the
    oracle, outputs, final state and every gradient, with a repeated state_map row."""
    B, H = 3, 2
    d = wkv6_inputs(B, T, H, N, dtype=dtype, seed=640 + T + N, n_state=2, with_grads=True)
    d["state_map"] = torch.tensor([1, 0, 1], dtype=torch.int32)
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rkvwu"}
    s0r = d["init_state"].float().clone().requires_grad_(True)
    y_ref, s_ref = OracleOp(N, T)(ref["r"], ref["k"], ref["v"], ref["w"], ref["u"], with_state=True,
                                  init_state=s0r, state_map=d["state_map"])
    ((y_ref * d["d_y"].float()).sum() + (s_ref * d["d_state"].float()).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].cuda().requires_grad_(True)
    y, s = ro.RWKV6_OP(N, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                             state_map=d["state_map"].cuda())
    assert y.shape == (B, T, H * N) and s.shape == (B, H, N, N) and y.dtype == dtype
    ((y.float() * d["d_y"].cuda().float()).sum() + (s.float() * d["d_state"].cuda().float()).sum()).backward()
    errs = {"y": rel_l2(y, y_ref), "s": rel_l2(s, s_ref), "ds0": rel_l2(s0.grad, s0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rkvwu"})
    assert all(e < tol for e in errs.values()), errs
    assert g["u"].grad.shape == d["u"].shape


def test_unsupported_head_size_raises():
    with pytest.raises(ValueError):
        ro.RWKV6_OP(48, 16)


def test_u_shapes_list_state_map_and_errors():
    B, T, H = 2, 12, 2
    d = wkv6_inputs(B, T, H, seed=61, n_state=3)
    x = {n: d[n].cuda() for n in "rkvw"}
    op = ro.RWKV6_OP(64, T)
    y0, s0 = op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), with_state=True, init_state=d["init_state"].cuda(),
                state_map=[2, 0])
    y1, s1 = op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda().reshape(1, 1, -1), with_state=True,
                init_state=d["init_state"].cuda(), state_map=torch.tensor([2, 0], dtype=torch.int64))
    assert torch.equal(y0, y1) and torch.equal(s0, s1)
    with pytest.raises(ValueError):
        op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), with_state=True, init_state=d["init_state"].cuda())
    with pytest.raises(AssertionError):
        op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), with_state=True, init_state=d["init_state"].cuda(),
           state_map=[0, 3])
    with pytest.raises(AssertionError):
        op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), state_map=[0, 1])
    # a single [H,N,N] state is shared by the batch
    y2, _ = op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), with_state=True, init_state=d["init_state"][1].cuda())
    y3, _ = op(x["r"], x["k"], x["v"], x["w"], d["u"].cuda(), with_state=True, init_state=d["init_state"].cuda(),
               state_map=[1, 1])
    assert torch.equal(y2, y3)


def test_split_sequence_equals_whole():
    B, T, H = 2, 150, 3
    d = wkv6_inputs(B, T, H, seed=62, n_state=B)
    x = {n: d[n].cuda() for n in "rkvw"}
    u = d["u"].cuda()
    op = ro.RWKV6_OP(64, T)
    y, s = op(x["r"], x["k"], x["v"], x["w"], u, with_state=True, init_state=d["init_state"].cuda())
    y1, s1 = op(*[x[n][:, :61] for n in "rkvw"], u, with_state=True, init_state=d["init_state"].cuda())
    y2, s2 = op(*[x[n][:, 61:] for n in "rkvw"], u, with_state=True, init_state=s1)
    assert rel_l2(torch.cat([y1, y2], 1), y) < 1e-5 and rel_l2(s2, s) < 1e-5


def test_full_size_sampled_units():
    """Benchmark configuration 4 at full size (fp32, B16 T4096 C2048, 4 initial states): sampled
    (batch, head) units against the oracle run on those units alone."""
    B, T, H = 16, 4096, 32
    d = wkv6_inputs(B, T, H, seed=1004, device="cuda", n_state=4, with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].requires_grad_(True)
    y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                              state_map=d["state_map"])
    ((y * d["d_y"]).sum() + (s * d["d_state"]).sum()).backward()
    units = [(0, 0), (5, 13), (15, 31)]
    smap = d["state_map"].cpu()
    for (b, h) in units:
        sl = slice(h * 64, (h + 1) * 64)
        sub = [g[n].detach()[b:b + 1, :, sl].cpu() for n in "rkvw"] + [g["u"].detach()[h:h + 1].cpu()]
        s0b = s0.detach()[smap[b]:smap[b] + 1, h:h + 1].cpu()
        y_ref, s_ref = OracleOp(64, T)(*sub, with_state=True, init_state=s0b)
        assert rel_l2(y[b:b + 1, :, sl], y_ref) < 1e-4
        assert rel_l2(s[b:b + 1, h:h + 1], s_ref) < 1e-4
        gr = wkv6_manual_backward(*sub, s0b, d["d_y"][b:b + 1, :, sl].cpu(), d["d_state"][b:b + 1, h:h + 1].cpu(), 64)
        for n, gn in zip("rkvw", gr[:4]):
            assert rel_l2(g[n].grad[b:b + 1, :, sl], gn) < 1e-4, n


def test_full_size_du_and_init_state_gradient():
    """Configuration 4 at full size: the two gradients that sum over batch rows.  du of one head (all 16
    batch rows and 4096 tokens) and the gradient of the initial-state table for that head (every table row is
    the start of several batch rows through state_map) against the float64 reverse recurrence."""
    B, T, H = 16, 4096, 32
    d = wkv6_inputs(B, T, H, seed=1004, device="cuda", n_state=4, with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].requires_grad_(True)
    y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                              state_map=d["state_map"])
    ((y * d["d_y"]).sum() + (s * d["d_state"]).sum()).backward()
    smap = d["state_map"].cpu().long()
    assert len(set(smap.tolist())) < B      # table rows are shared
    for h in (0, 19):
        sl = slice(h * 64, (h + 1) * 64)
        sub = [g[n].detach()[:, :, sl].cpu() for n in "rkvw"] + [g["u"].detach()[h:h + 1].cpu()]
        s0b = s0.detach()[:, h:h + 1].cpu()[smap]                      # [B,1,64,64]
        gr = wkv6_manual_backward(*sub, s0b, d["d_y"][:, :, sl].cpu(), d["d_state"][:, h:h + 1].cpu(), 64)
        assert rel_l2(g["u"].grad[h:h + 1], gr[4]) < 1e-4
        ds0_ref = torch.zeros(4, 1, 64, 64, dtype=gr[5].dtype).index_add_(0, smap, gr[5])
        assert rel_l2(s0.grad[:, h:h + 1], ds0_ref) < 1e-4


@pytest.mark.parametrize("T", [2, 3])
def test_very_short_sequences_with_fast_decays(T):
    """Two- and three-token sequences whose decays are fast (w ~ N(-0.3, 0.8^2)): the decay gradient is then a
    small remainder of sums that cancel, the case in which the tensor-core path's roundings would show most;
    such sequences take the recurrence.  Twelve seeds against the float64 oracle."""
    B, H = 2, 7
    for seed in range(12):
        d = wkv6_inputs(B, T, H, dtype=torch.float32, seed=7700 + seed, n_state=1, with_grads=True)
        g0 = torch.Generator().manual_seed(seed)
        d["w"] = -0.3 + 0.8 * torch.randn(d["w"].shape, generator=g0)
        ref = {n: d[n].double().clone().requires_grad_(True) for n in "rkvwu"}
        s0r = d["init_state"].double().clone().requires_grad_(True)
        y_ref, s_ref = OracleOp(64, T, compute_dtype=torch.float64)(ref["r"], ref["k"], ref["v"], ref["w"], ref["u"],
                                                                    with_state=True, init_state=s0r)
        ((y_ref * d["d_y"].double()).sum() + (s_ref * d["d_state"].double()).sum()).backward()
        g = {n: d[n].cuda().requires_grad_(True) for n in "rkvwu"}
        s0 = d["init_state"].cuda().requires_grad_(True)
        y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0)
        ((y * d["d_y"].cuda()).sum() + (s * d["d_state"].cuda()).sum()).backward()
        errs = {"y": rel_l2(y, y_ref), "s": rel_l2(s, s_ref), "ds0": rel_l2(s0.grad, s0r.grad)}
        errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rkvwu"})
        assert all(e < 1e-4 for e in errs.values()), (seed, errs)


@pytest.mark.parametrize("B,H,T", [(10, 20, 300), (150, 1, 512), (3, 50, 257), (9, 40, 1100), (20, 16, 520)])
def test_more_units_than_sms_work_items(B, H, T, monkeypatch):
    """With more (batch, head) units than CTA slots the chunked kernels work on every unit as several items
    (stretches of its chunks: two in the backward above 148 units, two or four in the forward above 296) and hand
    the state, or its gradient, from one to the next: outputs, gradients, du over all batch rows and the gradient
    of a shared initial-state table against the float32 recurrence."""
    d = wkv6_inputs(B, T, H, dtype=torch.float32, seed=31 + T, device="cuda", n_state=3, with_grads=True)
    res = {}
    for algo in ("chunked", "recurrent"):
        monkeypatch.setenv("RWKV_OPS_B200_WKV6_ALGO", algo)
        g = {n: d[n].clone().requires_grad_(True) for n in "rkvwu"}
        s0 = d["init_state"].clone().requires_grad_(True)
        y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                                  state_map=d["state_map"])
        torch.autograd.backward([y, s], [d["d_y"], d["d_state"]])
        res[algo] = {"y": y, "s": s, "ds0": s0.grad, **{n: g[n].grad for n in "rkvwu"}}
    errs = {k_: rel_l2(res["chunked"][k_], res["recurrent"][k_]) for k_ in res["chunked"]}
    assert max(errs.values()) < 1e-4, errs
