"""Packed variable-length batches against the CPU oracle run on every sequence alone."""
import pytest
import torch

import rwkv_ops_b200 as ro
from rwkv_ops_b200.workloads import rel_l2, rwkv7_inputs

pytestmark = pytest.mark.gpu

NAMES = "rwkvab"


def _oracle_per_sequence(d, cu, h0, d_out, d_state):
    """Outputs, final states and gradients of the oracle, sequence by sequence (float32, CPU)."""
    from oracle import generalized_delta_rule as oracle_gdr
    g = {n: d[n].detach().float().clone().requires_grad_(True) for n in NAMES}
    h = None if h0 is None else h0.detach().clone().requires_grad_(True)
    outs, states = [], []
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        hi = None if h is None else (h[i:i + 1] if h.shape[0] > 1 else h)
        o, st = oracle_gdr(*[g[n][:, s:e] for n in NAMES], initial_state=hi)
        outs.append(o)
        states.append(st)
    o, st = torch.cat(outs, 1), torch.cat(states, 0)
    ((o * d_out.float()).sum() + (st * d_state).sum()).backward()
    return o, st, {n: g[n].grad for n in NAMES}, (None if h is None else h.grad)


@pytest.mark.parametrize("lens,with_state,bcast", [
    ([64, 128, 64], False, False),            # whole chunks only
    ([1, 70, 5, 200, 64, 63], True, False),   # ragged: partial last chunks, a one-token sequence
    ([130, 17], True, True),                  # one initial state shared by the sequences
    ([333], True, False),                     # a single sequence
])
def test_varlen_forward_backward_matches_oracle(lens, with_state, bcast):
    from rwkv_ops_b200 import generalized_delta_rule_varlen
    H = 3
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = rwkv7_inputs(1, T, H, dtype=torch.bfloat16, seed=4242 + T)
    gen = torch.Generator().manual_seed(T)
    n_state = 1 if bcast else len(lens)
    h0 = 0.1 * torch.randn(n_state, H, 64, 64, generator=gen) if with_state else None
    d_out = torch.randn(1, T, H, 64, generator=gen).bfloat16()
    d_state = 0.1 * torch.randn(len(lens), H, 64, 64, generator=gen)
    o_ref, s_ref, g_ref, dh_ref = _oracle_per_sequence(d, cu, h0, d_out, d_state)

    g = {n: d[n].cuda().requires_grad_(True) for n in NAMES}
    h = None if h0 is None else h0.cuda().requires_grad_(True)
    o, st = generalized_delta_rule_varlen(*[g[n] for n in NAMES], torch.tensor(cu), initial_state=h)
    assert o.shape == (1, T, H, 64) and o.dtype == torch.bfloat16 and st.shape == (len(lens), H, 64, 64)
    assert rel_l2(o, o_ref) <= 2e-2
    assert rel_l2(st, s_ref) <= 2e-2
    torch.autograd.backward([o, st], [d_out.cuda(), d_state.cuda()])
    for n in NAMES:
        assert rel_l2(g[n].grad, g_ref[n]) <= 2e-2, n
    if h is not None:
        assert rel_l2(h.grad, dh_ref) <= 2e-2


def test_varlen_equals_dense_calls_and_leaves_no_gaps():
    """Same numbers as one dense call per sequence; every output row is written exactly once."""
    from rwkv_ops_b200 import generalized_delta_rule, generalized_delta_rule_varlen
    lens = [100, 64, 1, 257]
    H, T = 2, sum(lens)
    cu = [0, 100, 164, 165, 422]
    d = rwkv7_inputs(1, T, H, dtype=torch.bfloat16, seed=99, device="cuda")
    o, st = generalized_delta_rule_varlen(*[d[n] for n in NAMES], cu)
    from rwkv_ops_b200 import PackedSequences
    o2, st2 = generalized_delta_rule_varlen(*[d[n] for n in NAMES], PackedSequences(cu, "cuda"))
    assert torch.equal(o, o2) and torch.equal(st, st2)
    for i in range(len(lens)):
        s, e = cu[i], cu[i + 1]
        oi, si = generalized_delta_rule(*[d[n][:, s:e].contiguous() for n in NAMES])
        # same algorithm, separately compiled kernel variants: a few bfloat16 results differ by one ulp
        assert rel_l2(o[:, s:e], oi) <= 5e-3
        assert rel_l2(st[i:i + 1], si) <= 5e-3
    assert torch.isfinite(o.float()).all()


def test_varlen_long_sequences_forward_backward_equal_dense_calls():
    """Lengths in the thousands (more chunk slots than SMs, skipped slots, partial last chunks): outputs,
    states and every gradient equal those of one dense call per sequence (itself checked against the oracle)."""
    from rwkv_ops_b200 import generalized_delta_rule, generalized_delta_rule_varlen
    gen = torch.Generator().manual_seed(31)
    lens = torch.randint(50, 2500, (9,), generator=gen).tolist() + [4096, 1]
    H, T = 4, sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = rwkv7_inputs(1, T, H, dtype=torch.bfloat16, seed=123, device="cuda", with_grads=True)
    h0 = (0.1 * torch.randn(len(lens), H, 64, 64, device="cuda")).requires_grad_(True)
    d_state = 0.1 * torch.randn(len(lens), H, 64, 64, device="cuda")
    g = {n: d[n].clone().requires_grad_(True) for n in NAMES}
    o, st = generalized_delta_rule_varlen(*[g[n] for n in NAMES], cu, initial_state=h0)
    torch.autograd.backward([o, st], [d["d_out"], d_state])
    h0_ref = h0.detach().clone().requires_grad_(True)
    ref = {n: d[n].clone().requires_grad_(True) for n in NAMES}
    outs, states = [], []
    for i in range(len(lens)):
        s, e = cu[i], cu[i + 1]
        oi, si = generalized_delta_rule(*[ref[n][:, s:e] for n in NAMES], initial_state=h0_ref[i:i + 1])
        outs.append(oi)
        states.append(si)
    o_ref, s_ref = torch.cat(outs, 1), torch.cat(states, 0)
    torch.autograd.backward([o_ref, s_ref], [d["d_out"], d_state])
    assert rel_l2(o, o_ref) <= 5e-3 and rel_l2(st, s_ref) <= 5e-3
    for n in NAMES:
        assert rel_l2(g[n].grad, ref[n].grad) <= 1e-2, n
    assert rel_l2(h0.grad, h0_ref.grad) <= 1e-2


def test_varlen_float32_runs_per_sequence():
    from rwkv_ops_b200 import generalized_delta_rule_varlen
    lens = [9, 30]
    d = rwkv7_inputs(1, 39, 2, dtype=torch.float32, seed=5)
    from oracle import generalized_delta_rule as oracle_gdr
    refs = [oracle_gdr(*[d[n][:, s:e] for n in NAMES]) for s, e in ((0, 9), (9, 39))]
    o, st = generalized_delta_rule_varlen(*[d[n].cuda() for n in NAMES], [0, 9, 39])
    assert rel_l2(o, torch.cat([x[0] for x in refs], 1)) <= 1e-4
    assert rel_l2(st, torch.cat([x[1] for x in refs], 0)) <= 1e-4


def test_varlen_rejects_bad_arguments():
    from rwkv_ops_b200 import generalized_delta_rule_varlen
    d = rwkv7_inputs(1, 20, 2, dtype=torch.bfloat16, seed=6, device="cuda")
    x = [d[n] for n in NAMES]
    with pytest.raises(ValueError):
        generalized_delta_rule_varlen(*x, [0, 10, 19])         # does not end at the token count
    with pytest.raises(ValueError):
        generalized_delta_rule_varlen(*x, [0, 10, 10, 20])     # an empty sequence
    with pytest.raises(ValueError):
        generalized_delta_rule_varlen(*[t.expand(2, -1, -1, -1) for t in x], [0, 20])


@pytest.mark.parametrize("bcast", [False, True])
def test_varlen_with_decays_beyond_the_range_of_the_chunked_kernels(bcast):
    """Packed sequences of which some decay too fast for the tensor-core kernels (w ~ 1 + 0.3 N(0,1) in one
    sequence for all heads, and in one head of another): those (sequence, head) units are recomputed by the
    float32 recurrence inside the call, reading their tokens at the sequence's offset in the packed row."""
    from rwkv_ops_b200 import generalized_delta_rule_varlen
    H, lens = 3, [70, 131, 64, 200]
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = rwkv7_inputs(1, T, H, dtype=torch.bfloat16, seed=4343)
    gen = torch.Generator().manual_seed(11)
    fast = (1.0 + 0.3 * torch.randn(1, T, H, 64, generator=gen)).bfloat16()
    d["w"][:, cu[1]:cu[2]] = fast[:, cu[1]:cu[2]]              # sequence 1, every head
    d["w"][:, cu[3]:cu[4], 2] = fast[:, cu[3]:cu[4], 2]        # sequence 3, head 2
    n_state = 1 if bcast else len(lens)
    h0 = 0.1 * torch.randn(n_state, H, 64, 64, generator=gen)
    d_out = torch.randn(1, T, H, 64, generator=gen).bfloat16()
    d_state = 0.1 * torch.randn(len(lens), H, 64, 64, generator=gen)
    o_ref, s_ref, g_ref, dh_ref = _oracle_per_sequence(d, cu, h0, d_out, d_state)

    g = {n: d[n].cuda().requires_grad_(True) for n in NAMES}
    h = h0.cuda().requires_grad_(True)
    o, st = generalized_delta_rule_varlen(*[g[n] for n in NAMES], torch.tensor(cu), initial_state=h)
    torch.autograd.backward([o, st], [d_out.cuda(), d_state.cuda()])
    assert rel_l2(o, o_ref) <= 2e-2 and rel_l2(st, s_ref) <= 2e-2
    for n in NAMES:
        assert rel_l2(g[n].grad, g_ref[n]) <= 2e-2, n
    assert rel_l2(h.grad, dh_ref) <= 2e-2
    # sequence by sequence as well: a wrong token offset in one unit would hide in the norm of the whole row
    for i in range(len(lens)):
        sl = slice(cu[i], cu[i + 1])
        assert rel_l2(o[:, sl], o_ref[:, sl]) <= 2e-2, i
        for n in NAMES:
            assert rel_l2(g[n].grad[:, sl], g_ref[n][:, sl]) <= 2e-2, (i, n)


# ---------------------------------------------------------------------------------------------------------
# RWKV6 wkv on packed batches
# ---------------------------------------------------------------------------------------------------------
def _wkv6_packed_case(lens, H, dtype, seed, w_scale=None):
    from rwkv_ops_b200.workloads import wkv6_inputs
    total = sum(lens)
    d = wkv6_inputs(1, total, H, dtype=dtype, seed=seed, with_grads=True)
    g = torch.Generator().manual_seed(seed + 1)
    d["init_state"] = (0.1 * torch.randn(2, H, 64, 64, generator=g)).to(dtype)
    d["d_state"] = (0.1 * torch.randn(len(lens), H, 64, 64, generator=g)).to(dtype)
    if w_scale is not None:      # one head of one sequence decays faster than the tensor-core kernels' range
        w = d["w"].float().view(1, total, H, 64)
        s0 = sum(lens[:1])
        w[:, s0:s0 + lens[1], 0] = w_scale
        d["w"] = w.view(1, total, H * 64).to(dtype)
    return d


@pytest.mark.parametrize("lens,dtype,tol,w_scale", [
    ((70, 1, 64, 129, 5), torch.float32, 1e-4, None),
    ((70, 1, 64, 129, 5), torch.bfloat16, 2e-2, None),
    ((33, 200, 64), torch.float32, 1e-4, 1.2),      # exp(1.2) = 3.3 per token: far beyond the chunked range
])
def test_wkv6_packed_equals_per_sequence_oracle(lens, dtype, tol, w_scale):
    """``wkv6_varlen`` on sequences packed end to end against the CPU oracle run on every sequence alone:
    outputs, final states, and the gradients of r, k, v, w, u and of an initial-state table whose rows are
    shared between sequences."""
    from oracle import RWKVKernelOperator as OracleOp
    H = 2
    d = _wkv6_packed_case(lens, H, dtype, seed=8100 + len(lens), w_scale=w_scale)
    smap = [i % 2 for i in range(len(lens))]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    # oracle, sequence by sequence
    ref = {n: d[n].float().clone().requires_grad_(True) for n in "rkvwu"}
    s0r = d["init_state"].float().clone().requires_grad_(True)
    ys, ss = [], []
    for i, n in enumerate(lens):
        sl = slice(cu[i], cu[i + 1])
        yi, si = OracleOp(64, n)(ref["r"][:, sl], ref["k"][:, sl], ref["v"][:, sl], ref["w"][:, sl], ref["u"],
                                 with_state=True, init_state=s0r, state_map=torch.tensor([smap[i]], dtype=torch.int32))
        ys.append(yi)
        ss.append(si)
    y_ref, s_ref = torch.cat(ys, dim=1), torch.cat(ss, dim=0)
    ((y_ref * d["d_y"].float()).sum() + (s_ref * d["d_state"].float()).sum()).backward()
    # the packed operator
    g = {n: d[n].cuda().requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].cuda().requires_grad_(True)
    y, s = ro.wkv6_varlen(g["r"], g["k"], g["v"], g["w"], g["u"], cu, init_state=s0, state_map=smap)
    assert y.shape == d["r"].shape and y.dtype == dtype and s.shape == (len(lens), H, 64, 64)
    ((y.float() * d["d_y"].cuda().float()).sum() + (s.float() * d["d_state"].cuda().float()).sum()).backward()
    errs = {"y": rel_l2(y, y_ref), "s": rel_l2(s, s_ref), "ds0": rel_l2(s0.grad, s0r.grad)}
    errs.update({f"d{n}": rel_l2(g[n].grad, ref[n].grad) for n in "rkvwu"})
    assert all(e < tol for e in errs.values()), errs


def test_wkv6_packed_matches_dense_when_lengths_are_equal():
    """Two sequences of 128 tokens, packed and as a dense [2, 128, C] batch: the same kernels on the same data."""
    from rwkv_ops_b200.workloads import wkv6_inputs
    H, T = 2, 128
    d = wkv6_inputs(2, T, H, dtype=torch.float32, seed=8200)
    x = {n: d[n].cuda() for n in "rkvw"}
    u = d["u"].cuda()
    y_d, s_d = ro.RWKV6_OP(64, T)(x["r"], x["k"], x["v"], x["w"], u, with_state=True)
    p = {n: x[n].reshape(1, 2 * T, -1) for n in "rkvw"}
    y_p, s_p = ro.wkv6_varlen(p["r"], p["k"], p["v"], p["w"], u, [0, T, 2 * T])
    assert torch.equal(y_p.reshape(2, T, -1), y_d) and torch.equal(s_p, s_d)


def test_wkv6_packed_with_more_sequences_than_cta_slots():
    """400 sequences of one head, 1 .. 1100 tokens: the chunked kernels run them as work items on persistent CTAs
    (stretches of chunks with the state handed on; sequences shorter than the number of stretches have empty
    ones), against the recurrence run on every sequence alone."""
    import random
    from rwkv_ops_b200.workloads import wkv6_inputs
    rng = random.Random(4)
    n_seq = 400
    lens = [rng.choice([1, 5, 64, 100, 256, 300, 513, 1100]) for _ in range(n_seq)]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = wkv6_inputs(1, cu[-1], 1, dtype=torch.float32, seed=78, device="cuda", with_grads=True)
    d_state = 0.1 * torch.randn(n_seq, 1, 64, 64, device="cuda")
    g = {n: d[n].clone().requires_grad_(True) for n in "rkvwu"}
    y, s = ro.wkv6_varlen(g["r"], g["k"], g["v"], g["w"], g["u"], cu)
    torch.autograd.backward([y, s], [d["d_y"], d_state])
    g2 = {n: d[n].clone().requires_grad_(True) for n in "rkvwu"}
    import os
    old = os.environ.get("RWKV_OPS_B200_WKV6_ALGO")
    os.environ["RWKV_OPS_B200_WKV6_ALGO"] = "recurrent"
    try:
        ys, ss = [], []
        for i in range(n_seq):
            sl = slice(cu[i], cu[i + 1])
            yi, si = ro.RWKV6_OP(64, lens[i])(g2["r"][:, sl], g2["k"][:, sl], g2["v"][:, sl], g2["w"][:, sl], g2["u"],
                                              with_state=True)
            ys.append(yi)
            ss.append(si)
        torch.autograd.backward([torch.cat(ys, 1), torch.cat(ss, 0)], [d["d_y"], d_state])
    finally:
        if old is None:
            os.environ.pop("RWKV_OPS_B200_WKV6_ALGO")
        else:
            os.environ["RWKV_OPS_B200_WKV6_ALGO"] = old
    errs = {"y": rel_l2(y, torch.cat(ys, 1)), "s": rel_l2(s, torch.cat(ss, 0))}
    errs.update({n: rel_l2(g[n].grad, g2[n].grad) for n in "rkvwu"})
    assert max(errs.values()) < 1e-4, errs
