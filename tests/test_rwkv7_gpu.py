"""GPU parity of the RWKV7 generalized delta rule against the CPU oracle and the golden vectors
recorded from the reference's native operator.  Tolerances (relative L2 per tensor): 1e-4 for
float32 token tensors, 2e-2 for bfloat16 / float16, on outputs, states and every gradient."""
import glob
import os

import numpy as np
import pytest
import torch

import rwkv_ops_b200 as ro
from oracle import generalized_delta_rule as oracle_gdr, rwkv7_manual_backward
from rwkv_ops_b200.workloads import rwkv7_inputs, rwkv7_pad_lengths, apply_w_padding, rel_l2

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
R7 = sorted(glob.glob(os.path.join(GOLDEN, "rwkv7_*.npz")))
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
ALGOS = ["recurrent", "auto"]


@pytest.fixture(autouse=True)
def _need_cuda():
    assert torch.cuda.is_available(), "these tests need a CUDA device"


@pytest.fixture(params=ALGOS)
def algo(request, monkeypatch):
    monkeypatch.setenv("RWKV_OPS_B200_RWKV7_ALGO", request.param)
    return request.param


def _cuda(d, grad=False):
    out = {}
    for k_, t in d.items():
        t = t.cuda()
        if grad and t.is_floating_point() and k_ in ("r", "w", "k", "v", "a", "b", "initial_state"):
            t.requires_grad_(True)
        out[k_] = t
    return out


@pytest.mark.parametrize("path", R7, ids=[os.path.basename(p)[:-4] for p in R7])
def test_golden_forward_backward(path, algo):
    z = np.load(path)
    dt = getattr(torch, str(z["dtype"]))
    tol = TOL[dt]
    ins = {n: torch.from_numpy(z[f"in_{n}"]).to(dt).cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = torch.from_numpy(z["in_initial_state"]).cuda().requires_grad_(True) if "in_initial_state" in z else None
    o, s = ro.generalized_delta_rule(ins["r"], ins["w"], ins["k"], ins["v"], ins["a"], ins["b"], initial_state=h0)
    assert o.dtype == dt and s.dtype == torch.float32 and o.shape == ins["r"].shape
    assert rel_l2(o, torch.from_numpy(z["o"])) < tol
    assert rel_l2(s, torch.from_numpy(z["final_state"])) < tol
    loss = (o.float() * torch.from_numpy(z["d_out"]).cuda()).sum() + (s * torch.from_numpy(z["d_state"]).cuda()).sum()
    loss.backward()
    for n in "rwkvab":
        assert rel_l2(ins[n].grad, torch.from_numpy(z[f"grad_{n}"])) < tol, n
    if h0 is not None:
        assert rel_l2(h0.grad, torch.from_numpy(z["grad_initial_state"])) < tol


@pytest.mark.parametrize("T", [1, 2, 7, 15, 16, 17, 63, 64, 65, 130])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_lengths_vs_oracle(T, dtype, algo):
    B, H = 2, 3
    d = rwkv7_inputs(B, T, H, dtype=dtype, seed=500 + T, with_state=True, with_grads=True)
    ref_in = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[ref_in[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref.float() * d["d_out"].float()).sum() + (s_ref * d["d_state"]).sum()).backward()

    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    ((o.float() * d["d_out"].cuda().float()).sum() + (s * d["d_state"].cuda()).sum()).backward()
    tol = TOL[dtype]
    assert rel_l2(o, o_ref) < tol and rel_l2(s, s_ref) < tol
    for n in "rwkvab":
        assert rel_l2(g[n].grad, ref_in[n].grad) < tol, n
    assert rel_l2(h0.grad, h0r.grad) < tol


def test_broadcast_state_no_state_and_bare_output(algo):
    B, T, H = 3, 21, 2
    d = rwkv7_inputs(B, T, H, seed=77, with_state=True, n_state=1, with_grads=True)
    ref_in = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[ref_in[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref * d["d_out"]).sum() + (s_ref * d["d_state"]).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    ((o * d["d_out"].cuda()).sum() + (s * d["d_state"].cuda()).sum()).backward()
    assert h0.grad.shape == (1, H, 64, 64)
    assert rel_l2(o, o_ref) < 1e-4 and rel_l2(s, s_ref) < 1e-4 and rel_l2(h0.grad, h0r.grad) < 1e-4
    for n in "rwkvab":
        assert rel_l2(g[n].grad, ref_in[n].grad) < 1e-4, n
    # no initial state; output_final_state=False returns a bare tensor
    o2 = ro.generalized_delta_rule(*[d[n].cuda() for n in "rwkvab"], output_final_state=False)
    assert torch.is_tensor(o2)
    assert rel_l2(o2, oracle_gdr(*[d[n] for n in "rwkvab"], output_final_state=False)) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_first_is_a_permutation(dtype, algo):
    B, T, H = 2, 37, 3
    d = rwkv7_inputs(B, T, H, dtype=dtype, seed=78, with_state=True, with_grads=True)
    base = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    o, s = ro.generalized_delta_rule(*[base[n] for n in "rwkvab"], initial_state=d["initial_state"].cuda())
    (o.float() * d["d_out"].cuda().float()).sum().backward()
    hf = {n: d[n].cuda().permute(0, 2, 1, 3).contiguous().requires_grad_(True) for n in "rwkvab"}
    o_hf, s_hf = ro.generalized_delta_rule(*[hf[n] for n in "rwkvab"], initial_state=d["initial_state"].cuda(),
                                           head_first=True)
    assert o_hf.shape == (B, H, T, 64)
    (o_hf.float() * d["d_out"].cuda().permute(0, 2, 1, 3).float()).sum().backward()
    assert torch.equal(o_hf.permute(0, 2, 1, 3), o) and torch.equal(s_hf, s)
    for n in "rwkvab":
        assert torch.equal(hf[n].grad.permute(0, 2, 1, 3), base[n].grad), n


def test_padding_recipe_leaves_state_unchanged(algo):
    """The reference's padding check (test_script/test_rwkv7_value.py:210-229): doubling T with
    w += -1e9 and the other inputs zeroed on the tail must leave the final state bit-identical."""
    B, T, H = 2, 48, 2
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=79)
    x = {n: d[n].cuda() for n in "rwkvab"}
    _, s = ro.generalized_delta_rule(*[x[n] for n in "rwkvab"])
    pad = {n: torch.cat([x[n], torch.zeros_like(x[n])], dim=1) for n in "rwkvab"}
    lengths = torch.full((B,), T)
    pad["w"] = apply_w_padding(pad["w"], lengths)
    o2, s2 = ro.generalized_delta_rule(*[pad[n] for n in "rwkvab"])
    assert torch.equal(s, s2)
    assert torch.isfinite(o2).all()


def test_decode_steps_match_oracle_and_chain():
    """T == 1 goes through the dedicated step kernel; 24 chained steps equal one 24-token call."""
    B, T, H = 5, 24, 4
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=80, with_state=True)
    o_ref, s_ref = oracle_gdr(*[d[n] for n in "rwkvab"], initial_state=d["initial_state"])
    x = {n: d[n].cuda() for n in "rwkvab"}
    s = d["initial_state"].cuda()
    outs = []
    for t in range(T):
        o_t, s = ro.generalized_delta_rule(*[x[n][:, t:t + 1] for n in "rwkvab"], initial_state=s)
        outs.append(o_t)
    o = torch.cat(outs, dim=1)
    assert rel_l2(o, o_ref) < 2e-2 and rel_l2(s, s_ref) < 1e-4
    # the same 24 tokens in one call (bf16 tokens: chunked tensor-core path, bf16 tolerance)
    o_all, s_all = ro.generalized_delta_rule(*[x[n] for n in "rwkvab"], initial_state=d["initial_state"].cuda())
    assert rel_l2(s, s_all) < 2e-2 and rel_l2(o, o_all) < 2e-2


def test_step_kernel_in_place_through_c_abi():
    """Direct C-ABI call of the step entry point with state_out aliasing state_in."""
    from rwkv_ops_b200 import _lib
    lib = _lib.load()
    B, H = 7, 5
    d = rwkv7_inputs(B, 1, H, dtype=torch.float32, seed=81, with_state=True)
    x = {n: d[n].cuda().reshape(B, H, 64).contiguous() for n in "rwkvab"}
    s = d["initial_state"].cuda().clone()
    o = torch.empty(B, H, 64, device="cuda")
    rc = lib.rwkvb200_rwkv7_step(*[x[n].data_ptr() for n in "rwkvab"], s.data_ptr(), B, s.data_ptr(), o.data_ptr(),
                                 B, H, 64, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    o_ref, s_ref = oracle_gdr(*[d[n] for n in "rwkvab"], initial_state=d["initial_state"])
    assert rel_l2(o, o_ref.reshape(B, H, 64)) < 1e-5 and rel_l2(s, s_ref) < 1e-5


def test_split_sequence_equals_whole(algo):
    """Size-independent property: running T as two halves with the state handed over equals one run."""
    B, T, H = 2, 200, 2
    d = rwkv7_inputs(B, T, H, seed=82, with_state=True)
    x = {n: d[n].cuda() for n in "rwkvab"}
    h0 = d["initial_state"].cuda()
    o, s = ro.generalized_delta_rule(*[x[n] for n in "rwkvab"], initial_state=h0)
    o1, s1 = ro.generalized_delta_rule(*[x[n][:, :77] for n in "rwkvab"], initial_state=h0)
    o2, s2 = ro.generalized_delta_rule(*[x[n][:, 77:] for n in "rwkvab"], initial_state=s1)
    assert rel_l2(torch.cat([o1, o2], 1), o) < 1e-5 and rel_l2(s2, s) < 1e-5


@pytest.mark.parametrize("cfg", ["cfg1"])
def test_full_size_sampled_units(cfg, algo):
    """Benchmark configuration 1 at full size (bf16, B8 T4096 H32): outputs, final state and all six
    gradients of sampled (batch, head) units against the float32 oracle run on those units alone
    (units are independent recurrences)."""
    B, T, H = 8, 4096, 32
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=1001, device="cuda", with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"])
    ((o.float() * d["d_out"].float()).sum() + (s * d["d_state"]).sum()).backward()
    units = [(0, 0), (3, 17), (7, 31)]
    bi = torch.tensor([u[0] for u in units]); hi = torch.tensor([u[1] for u in units])

    def pick(t):   # [B,T,H,K] -> [n,T,1,K]
        return t.detach()[bi.cuda(), :, hi.cuda()].unsqueeze(2).cpu()

    sub = {n: pick(g[n]) for n in "rwkvab"}
    o_ref, s_ref = oracle_gdr(*[sub[n] for n in "rwkvab"])
    grads = rwkv7_manual_backward(*[sub[n] for n in "rwkvab"], None, pick(d["d_out"]),
                                  d["d_state"][bi.cuda(), hi.cuda()].unsqueeze(1).cpu())
    assert rel_l2(pick(o), o_ref) < 2e-2
    assert rel_l2(s[bi.cuda(), hi.cuda()].unsqueeze(1), s_ref) < 2e-2
    for n, gr in zip("rwkvab", grads[:6]):
        assert rel_l2(pick(g[n].grad), gr) < 2e-2, n


@pytest.mark.parametrize("T", [1, 37, 130])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_head_size_128_forward_backward(T, dtype, tol):
    """Head size 128, the size of the reference's own value test (test_script/test_rwkv7_value.py:46-51):
    outputs, final state and all gradients against the oracle."""
    B, H, K = 2, 3, 128
    fn, use_kernel = ro.get_generalized_delta_rule(HEAD_SIZE=K)
    assert use_kernel
    d = rwkv7_inputs(B, T, H, K, dtype=dtype, seed=900 + T, with_state=True, with_grads=True)
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[ref[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref * d["d_out"].float()).sum() + (s_ref * d["d_state"]).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = fn(*[g[n] for n in "rwkvab"], initial_state=h0)
    assert o.shape == (B, T, H, K) and o.dtype == dtype and s.shape == (B, H, K, K)
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    errs = {"o": rel_l2(o, o_ref), "s": rel_l2(s, s_ref), "dh0": rel_l2(h0.grad, h0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rwkvab"})
    assert all(e < tol for e in errs.values()), errs
    # [B, H, T, K] in and out
    with torch.no_grad():
        o_hf = fn(*[g[n].detach().permute(0, 2, 1, 3).contiguous() for n in "rwkvab"], initial_state=h0.detach(),
                  output_final_state=False, head_first=True)
    assert torch.equal(o_hf.permute(0, 2, 1, 3), o)


def test_one_token_without_state_has_no_decay_gradient():
    """One token and no initial state: the output does not depend on the decay, so dw is exactly zero (on the
    tensor-core path it would be the rounding residue of two chunk sums that cancel; sequences this short take
    the recurrence)."""
    B, T, H = 3, 1, 5
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=4242, with_grads=True)
    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"])
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    assert torch.count_nonzero(g["w"].grad) == 0
    assert torch.isfinite(g["r"].grad.float()).all() and torch.count_nonzero(g["k"].grad) > 0


def test_float32_tokens_on_the_tensor_core_path_by_request(monkeypatch):
    """RWKV_OPS_B200_RWKV7_ALGO=chunked with float32 tokens: rounded to bfloat16 for the tensor-core kernels,
    outputs and gradients back in float32, bfloat16-grade agreement with the oracle."""
    monkeypatch.setenv("RWKV_OPS_B200_RWKV7_ALGO", "chunked")
    B, T, H = 2, 150, 3
    d = rwkv7_inputs(B, T, H, dtype=torch.float32, seed=4343, with_state=True, with_grads=True)
    ref = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[ref[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref * d["d_out"]).sum() + (s_ref * d["d_state"]).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    assert o.dtype == torch.float32
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    errs = {"o": rel_l2(o, o_ref), "s": rel_l2(s, s_ref), "dh0": rel_l2(h0.grad, h0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rwkvab"})
    assert all(g[n].grad.dtype == torch.float32 for n in "rwkvab")
    assert all(e < 2e-2 for e in errs.values()), errs
    assert errs["o"] > 1e-5      # the bfloat16 path did run (the recurrence is float32-exact)
