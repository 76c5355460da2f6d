"""Delta rule with fused producers: bit-equal to the unfused operator, gradients against autograd through
the unfused formula (CPU oracle)."""
import pytest
import torch

from rwkv_ops_b200.workloads import rel_l2

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, seed, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = {n: torch.randn(B, T, H, 64, generator=g).bfloat16().to(device) for n in ("r", "w_pre", "k", "v", "kk_pre", "a_pre")}
    x["d_out"] = torch.randn(B, T, H, 64, generator=g).bfloat16().to(device)
    x["d_state"] = (0.1 * torch.randn(B, H, 64, 64, generator=g)).to(device)
    x["h0"] = (0.1 * torch.randn(B, H, 64, 64, generator=g)).to(device)
    return x


NAMES = ("r", "w_pre", "k", "v", "kk_pre", "a_pre")


@pytest.mark.parametrize("B,T,H", [(2, 64, 2), (1, 200, 3), (3, 37, 1)])
def test_fused_equals_unfused_operator_bitwise(B, T, H):
    from rwkv_ops_b200 import generalized_delta_rule, generalized_delta_rule_fused
    from rwkv_ops_b200.fused import producers
    x = _inputs(B, T, H, 11 * T, "cuda")
    o, s = generalized_delta_rule_fused(*[x[n] for n in NAMES], initial_state=x["h0"])
    w, a, b = producers(x["w_pre"], x["kk_pre"], x["a_pre"])
    o2, s2 = generalized_delta_rule(x["r"], w, x["k"], x["v"], a, b, initial_state=x["h0"])
    # the kernel's sigmoid and normalisation are not torch's: allow the last bfloat16 bit of w, a, b to differ
    assert rel_l2(o, o2) <= 5e-3 and rel_l2(s, s2) <= 5e-3


@pytest.mark.parametrize("B,T,H,with_state", [(2, 96, 2, True), (1, 150, 2, False)])
def test_fused_forward_backward_matches_oracle(B, T, H, with_state):
    from oracle import generalized_delta_rule as oracle_gdr
    from rwkv_ops_b200 import generalized_delta_rule_fused
    from rwkv_ops_b200.fused import W_SCALE
    x = _inputs(B, T, H, 5 + T)
    ref = {n: x[n].float().clone().requires_grad_(True) for n in NAMES}
    h_ref = x["h0"].clone().requires_grad_(True) if with_state else None
    w = W_SCALE * torch.sigmoid(ref["w_pre"])
    kk = torch.nn.functional.normalize(ref["kk_pre"], dim=-1, eps=1e-12)
    o_ref, s_ref = oracle_gdr(ref["r"], w, ref["k"], ref["v"], -kk, kk * torch.sigmoid(ref["a_pre"]),
                              initial_state=h_ref)
    ((o_ref * x["d_out"].float()).sum() + (s_ref * x["d_state"]).sum()).backward()

    g = {n: x[n].cuda().requires_grad_(True) for n in NAMES}
    h = x["h0"].cuda().requires_grad_(True) if with_state else None
    o, s = generalized_delta_rule_fused(*[g[n] for n in NAMES], initial_state=h)
    assert o.dtype == torch.bfloat16 and o.shape == (B, T, H, 64)
    torch.autograd.backward([o, s], [x["d_out"].cuda(), x["d_state"].cuda()])
    assert rel_l2(o, o_ref) <= 2e-2 and rel_l2(s, s_ref) <= 2e-2
    for n in NAMES:
        assert rel_l2(g[n].grad, ref[n].grad) <= 2e-2, n
    if with_state:
        assert rel_l2(h.grad, h_ref.grad) <= 2e-2


def test_fused_keep_and_recompute_agree(monkeypatch):
    from rwkv_ops_b200 import generalized_delta_rule_fused
    x = _inputs(2, 130, 2, 3, "cuda")
    grads = []
    for limit in (None, "0"):
        if limit is not None:
            monkeypatch.setenv("RWKV_OPS_B200_KEEP_LIMIT_MB", limit)
        g = {n: x[n].clone().requires_grad_(True) for n in NAMES}
        o, s = generalized_delta_rule_fused(*[g[n] for n in NAMES])
        torch.autograd.backward([o, s], [x["d_out"], x["d_state"]])
        grads.append([g[n].grad for n in NAMES])
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_fused_falls_back_for_float32():
    from rwkv_ops_b200 import generalized_delta_rule, generalized_delta_rule_fused
    from rwkv_ops_b200.fused import producers
    x = {n: t.float() for n, t in _inputs(1, 20, 2, 9, "cuda").items()}
    o, s = generalized_delta_rule_fused(*[x[n] for n in NAMES])
    w, a, b = producers(x["w_pre"], x["kk_pre"], x["a_pre"])
    o2, s2 = generalized_delta_rule(x["r"], w, x["k"], x["v"], a, b)
    assert torch.equal(o, o2) and torch.equal(s, s2)
