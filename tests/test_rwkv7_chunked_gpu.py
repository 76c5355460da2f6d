"""The chunked tcgen05 path of the RWKV7 delta rule (bf16 tokens) against the float32 CPU oracle.
Tolerance: relative L2 <= 2e-2 per tensor (the bar for bf16 inputs), and no bounded wait may run out."""
import pytest
import torch

import rwkv_ops_b200 as ro
from oracle import generalized_delta_rule as oracle_gdr
from rwkv_ops_b200 import _lib
from rwkv_ops_b200.workloads import rwkv7_inputs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _chunked(monkeypatch):
    monkeypatch.setenv("RWKV_OPS_B200_RWKV7_ALGO", "chunked")
    yield
    torch.cuda.synchronize()
    assert _lib.load().rwkvb200_device_status(1) == 0, "a bounded wait ran out inside a tensor-core kernel"


@pytest.mark.parametrize("T", [64, 128, 17, 65, 130, 257])
@pytest.mark.parametrize("state", [False, True])
def test_forward_vs_oracle(T, state):
    B, H = 2, 3
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=700 + T, with_state=state)
    h0 = d.get("initial_state")
    o_ref, s_ref = oracle_gdr(*[d[n] for n in "rwkvab"], initial_state=h0)
    with torch.no_grad():
        o, s = ro.generalized_delta_rule(*[d[n].cuda() for n in "rwkvab"],
                                         initial_state=None if h0 is None else h0.cuda())
    assert o.dtype == torch.bfloat16 and s.dtype == torch.float32
    assert rel_l2(o, o_ref) < 2e-2, rel_l2(o, o_ref)
    assert rel_l2(s, s_ref) < 2e-2, rel_l2(s, s_ref)


def test_forward_head_first_and_broadcast_state():
    B, T, H = 2, 100, 2
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=71, with_state=True, n_state=1)
    o_ref, s_ref = oracle_gdr(*[d[n] for n in "rwkvab"], initial_state=d["initial_state"])
    with torch.no_grad():
        o, s = ro.generalized_delta_rule(*[d[n].cuda().permute(0, 2, 1, 3).contiguous() for n in "rwkvab"],
                                         initial_state=d["initial_state"].cuda(), head_first=True)
    assert rel_l2(o.permute(0, 2, 1, 3), o_ref) < 2e-2 and rel_l2(s, s_ref) < 2e-2


def test_forward_full_size_sampled_units():
    """Configuration 1 (bf16, B8 T4096 H32) at full size against the oracle on sampled units."""
    B, T, H = 8, 4096, 32
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=1001, device="cuda")
    with torch.no_grad():
        o, s = ro.generalized_delta_rule(*[d[n] for n in "rwkvab"])
    for (b, h) in [(0, 0), (3, 17), (7, 31)]:
        sub = [d[n][b:b + 1, :, h:h + 1].cpu() for n in "rwkvab"]
        o_ref, s_ref = oracle_gdr(*sub)
        assert rel_l2(o[b:b + 1, :, h:h + 1], o_ref) < 2e-2
        assert rel_l2(s[b:b + 1, h:h + 1], s_ref) < 2e-2


@pytest.mark.parametrize("T", [64, 128, 17, 65, 130, 257])
@pytest.mark.parametrize("state", [False, True])
def test_backward_vs_oracle(T, state):
    B, H = 2, 3
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=800 + T, with_state=state, with_grads=True)
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    h0r = d["initial_state"].clone().requires_grad_(True) if state else None
    o_ref, s_ref = oracle_gdr(*[ref[n] for n in "rwkvab"], initial_state=h0r)
    ((o_ref * d["d_out"].float()).sum() + (s_ref * d["d_state"]).sum()).backward()
    g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True) if state else None
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    errs = {f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rwkvab"}
    if state:
        errs["dh0"] = rel_l2(h0.grad, h0r.grad)
    assert all(e < 2e-2 for e in errs.values()), errs


def test_backward_full_size_sampled_units():
    """Configuration 1 at full size: all six gradients of sampled (batch, head) units against the
    hand-derived float64 reverse recurrence of the oracle."""
    from oracle import rwkv7_manual_backward
    B, T, H = 8, 4096, 32
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=1001, device="cuda", with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"])
    torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])
    for (b, h) in [(0, 0), (5, 9), (7, 31)]:
        sub = [g[n].detach()[b:b + 1, :, h:h + 1].cpu() for n in "rwkvab"]
        grads = rwkv7_manual_backward(*sub, None, d["d_out"][b:b + 1, :, h:h + 1].cpu(),
                                      d["d_state"][b:b + 1, h:h + 1].cpu())
        errs = {n: rel_l2(g[n].grad[b:b + 1, :, h:h + 1], gr) for n, gr in zip("rwkvab", grads[:6])}
        assert all(e < 2e-2 for e in errs.values()), errs


def test_kept_tiles_and_recompute_agree(monkeypatch):
    """A training forward hands its per-chunk tiles to the backward; with the limit at zero the backward
    recomputes them from the inputs.  Both give the same gradients, and a second backward through the
    same graph works."""
    B, T, H = 2, 200, 2
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=91, with_state=True, with_grads=True)

    def run():
        g = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
        h0 = d["initial_state"].cuda().requires_grad_(True)
        o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
        torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()], retain_graph=True)
        first = [g[n].grad.clone() for n in "rwkvab"] + [h0.grad.clone()]
        for t in list(g.values()) + [h0]:
            t.grad = None
        torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
        second = [g[n].grad for n in "rwkvab"] + [h0.grad]
        return o, s, first, second

    o1, s1, kept_first, kept_second = run()
    monkeypatch.setenv("RWKV_OPS_B200_KEEP_LIMIT_MB", "0")
    o2, s2, rec_first, _ = run()
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    for a_, b_, c_ in zip(kept_first, kept_second, rec_first):
        assert torch.equal(a_, b_) and torch.equal(a_, c_)


def test_cfg2_full_size_padded_with_state():
    """Configuration 2 at full size (bf16, B16 T8192 H64, per-sequence initial state, trailing 0..512
    tokens of every sequence padded through w += -1e9): outputs, final state and gradients of sampled
    (batch, head) units against the oracle run on those units alone."""
    from oracle import rwkv7_manual_backward
    from rwkv_ops_b200.workloads import rwkv7_pad_lengths, apply_w_padding
    B, T, H = 16, 8192, 64
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=1002, device="cuda", with_state=True, with_grads=True)
    lengths = rwkv7_pad_lengths(B, T, seed=1002)
    d["w"] = apply_w_padding(d["w"], lengths)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0)
    torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])
    assert torch.isfinite(o).all() and torch.isfinite(s).all()
    for (b, h) in [(0, 0), (9, 33), (15, 63)]:
        sub = [g[n].detach()[b:b + 1, :, h:h + 1].cpu() for n in "rwkvab"]
        h0s = h0.detach()[b:b + 1, h:h + 1].cpu()
        o_ref, s_ref = oracle_gdr(*sub, initial_state=h0s)
        assert rel_l2(o[b:b + 1, :, h:h + 1], o_ref) < 2e-2
        assert rel_l2(s[b:b + 1, h:h + 1], s_ref) < 2e-2
        grads = rwkv7_manual_backward(*sub, h0s, d["d_out"][b:b + 1, :, h:h + 1].cpu(),
                                      d["d_state"][b:b + 1, h:h + 1].cpu())
        errs = {n: rel_l2(g[n].grad[b:b + 1, :, h:h + 1], gr) for n, gr in zip("rwkvab", grads[:6])}
        errs["h0"] = rel_l2(h0.grad[b:b + 1, h:h + 1], grads[6])
        assert all(e < 2e-2 for e in errs.values()), errs
