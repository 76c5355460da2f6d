"""Randomised cross-checks between independent paths of the library, all on the GPU: the tensor-core kernels
against the float32 recurrences, and the packed operators against one dense call per sequence.  Shapes, lengths
(1 .. 1500 tokens, around the 64-token chunk boundaries), decay distributions (the benchmark's, wide ones that mix
in-range and out-of-range channels, one fast head), state tables and layouts are drawn from a seeded generator.
Tolerances: relative L2 2e-2 for bfloat16 tokens, 1e-4 for float32 tokens."""
import random

import pytest
import torch

import rwkv_ops_b200 as ro
from rwkv_ops_b200.workloads import rel_l2, rwkv7_inputs, wkv6_inputs

pytestmark = pytest.mark.gpu

T_CHOICES = [1, 2, 3, 7, 8, 31, 63, 64, 65, 127, 128, 129, 200, 511, 777, 1024, 1500]


def _rwkv7(d, algo, monkeypatch, **kw):
    monkeypatch.setenv("RWKV_OPS_B200_RWKV7_ALGO", algo)
    g = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True) if "initial_state" in d else None
    o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=h0, **kw)
    torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])
    out = {"o": o, "s": s, **{f"d{n}": g[n].grad for n in "rwkvab"}}
    if h0 is not None:
        out["dh0"] = h0.grad
    return out


def _wkv6(d, algo, monkeypatch):
    monkeypatch.setenv("RWKV_OPS_B200_WKV6_ALGO", algo)
    g = {n: d[n].clone().requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].clone().requires_grad_(True) if "init_state" in d else None
    T = d["r"].shape[1]
    y, s = ro.RWKV6_OP(64, T)(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0,
                              state_map=d.get("state_map"))
    torch.autograd.backward([y, s], [d["d_y"], d["d_state"]])
    out = {"y": y, "s": s, **{f"d{n}": g[n].grad for n in "rkvwu"}}
    if s0 is not None:
        out["ds0"] = s0.grad
    return out


@pytest.mark.parametrize("seed", [1, 2])
def test_tensor_core_paths_against_the_recurrences(seed, monkeypatch):
    rng = random.Random(seed)
    for _ in range(40):
        B, H, T = rng.choice([1, 1, 2, 3, 5, 9]), rng.choice([1, 2, 3, 7, 16, 40]), rng.choice(T_CHOICES)
        if B * H * T > 600000:
            T = max(1, 600000 // (B * H))
        s = rng.randrange(1 << 30)
        # RWKV7, bfloat16 tokens
        with_state = rng.random() < 0.6
        d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=s, device="cuda", with_state=with_state,
                         n_state=rng.choice([1, B]) if with_state else None, with_grads=True)
        kind = rng.choice(["benchmark", "benchmark", "wide", "one_fast_head"])
        if kind == "wide":
            d["w"] = (-0.5 + 1.2 * torch.randn(d["w"].shape, device="cuda")).bfloat16()
        elif kind == "one_fast_head":
            w = d["w"].float()
            w[rng.randrange(B), :, rng.randrange(H)] = 1.3
            d["w"] = w.bfloat16()
        head_first = rng.random() < 0.25
        if head_first:
            for n in ("r", "w", "k", "v", "a", "b", "d_out"):
                d[n] = d[n].permute(0, 2, 1, 3).contiguous()
        a = _rwkv7(d, "chunked", monkeypatch, head_first=head_first)
        b = _rwkv7(d, "recurrent", monkeypatch, head_first=head_first)
        errs = {k: rel_l2(a[k], b[k]) for k in a}
        assert all(torch.isfinite(v.float()).all() for v in a.values()), (B, T, H, s, kind)
        assert max(errs.values()) < 2e-2, (dict(B=B, T=T, H=H, seed=s, kind=kind, head_first=head_first), errs)
        # wkv6, float32 tokens
        n_st = rng.choice([None, 1, 2, B])
        d6 = wkv6_inputs(B, T, H, dtype=torch.float32, seed=s + 1, device="cuda", n_state=n_st, with_grads=True)
        if rng.random() < 0.3:
            d6["w"] = -0.3 + 0.8 * torch.randn(d6["w"].shape, device="cuda")
        if n_st == B and rng.random() < 0.5:
            d6.pop("state_map")
        a = _wkv6(d6, "chunked", monkeypatch)
        b = _wkv6(d6, "recurrent", monkeypatch)
        errs = {k: rel_l2(a[k], b[k]) for k in a}
        assert max(errs.values()) < 1e-4, (dict(B=B, T=T, H=H, seed=s, n_state=n_st), errs)


def test_packed_operators_against_one_dense_call_per_sequence():
    rng = random.Random(5)
    for _ in range(25):
        H, n_seq = rng.choice([1, 2, 5, 12]), rng.choice([1, 2, 3, 6])
        lens = [rng.choice([1, 2, 5, 8, 9, 63, 64, 65, 100, 128, 130, 300, 513]) for _ in range(n_seq)]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        total, s = cu[-1], rng.randrange(1 << 30)
        # RWKV7
        d = rwkv7_inputs(1, total, H, dtype=torch.bfloat16, seed=s, device="cuda", with_grads=True)
        h0 = 0.1 * torch.randn(rng.choice([1, n_seq]), H, 64, 64, device="cuda") if rng.random() < 0.5 else None
        d_state = 0.1 * torch.randn(n_seq, H, 64, 64, device="cuda")
        g = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
        hp = h0.clone().requires_grad_(True) if h0 is not None else None
        o, st = ro.generalized_delta_rule_varlen(*[g[n] for n in "rwkvab"], cu, initial_state=hp)
        torch.autograd.backward([o, st], [d["d_out"], d_state])
        g2 = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
        hd = h0.clone().requires_grad_(True) if h0 is not None else None
        outs, sts = [], []
        for i in range(n_seq):
            sl = slice(cu[i], cu[i + 1])
            hi = None if hd is None else (hd[i:i + 1] if hd.shape[0] == n_seq else hd)
            oi, si = ro.generalized_delta_rule(*[g2[n][:, sl] for n in "rwkvab"], initial_state=hi)
            outs.append(oi)
            sts.append(si)
        torch.autograd.backward([torch.cat(outs, 1), torch.cat(sts, 0)], [d["d_out"], d_state])
        errs = {"o": rel_l2(o, torch.cat(outs, 1)), "s": rel_l2(st, torch.cat(sts, 0))}
        errs.update({n: rel_l2(g[n].grad, g2[n].grad) for n in "rwkvab"})
        if h0 is not None:
            errs["dh0"] = rel_l2(hp.grad, hd.grad)
        assert max(errs.values()) < 1e-3, (lens, H, s, errs)
        # wkv6
        d6 = wkv6_inputs(1, total, H, dtype=torch.float32, seed=s + 1, device="cuda", with_grads=True)
        n_st = rng.choice([None, 1, 2])
        s0 = 0.1 * torch.randn(n_st, H, 64, 64, device="cuda") if n_st else None
        smap = [rng.randrange(n_st) for _ in range(n_seq)] if n_st else None
        g = {n: d6[n].clone().requires_grad_(True) for n in "rkvwu"}
        sp = s0.clone().requires_grad_(True) if n_st else None
        y, st = ro.wkv6_varlen(g["r"], g["k"], g["v"], g["w"], g["u"], cu, init_state=sp, state_map=smap)
        torch.autograd.backward([y, st], [d6["d_y"], d_state])
        g2 = {n: d6[n].clone().requires_grad_(True) for n in "rkvwu"}
        sd = s0.clone().requires_grad_(True) if n_st else None
        ys, sts = [], []
        for i in range(n_seq):
            sl = slice(cu[i], cu[i + 1])
            kw = dict(init_state=sd, state_map=[smap[i]]) if n_st else {}
            yi, si = ro.RWKV6_OP(64, lens[i])(g2["r"][:, sl], g2["k"][:, sl], g2["v"][:, sl], g2["w"][:, sl], g2["u"],
                                              with_state=True, **kw)
            ys.append(yi)
            sts.append(si)
        torch.autograd.backward([torch.cat(ys, 1), torch.cat(sts, 0)], [d6["d_y"], d_state])
        errs = {"y": rel_l2(y, torch.cat(ys, 1)), "s": rel_l2(st, torch.cat(sts, 0))}
        errs.update({n: rel_l2(g[n].grad, g2[n].grad) for n in "rkvwu"})
        if n_st:
            errs["ds0"] = rel_l2(sp.grad, sd.grad)
        assert max(errs.values()) < 1e-5, (lens, H, s, n_st, errs)
