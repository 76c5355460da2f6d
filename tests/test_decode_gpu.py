"""In-place single-token decoding (Rwkv7DecodeState) against the CPU oracle run over the whole sequence."""
import pytest
import torch

from rwkv_ops_b200.workloads import rel_l2, rwkv7_inputs

pytestmark = pytest.mark.gpu


def _oracle(d, T):
    from oracle import generalized_delta_rule as oracle_gdr
    return oracle_gdr(*[d[n].float() for n in "rwkvab"], initial_state=d.get("initial_state"))


@pytest.mark.parametrize("dtype,state_dtype,tol", [
    (torch.float32, torch.float32, 1e-4),
    (torch.bfloat16, torch.float32, 2e-2),
    (torch.bfloat16, torch.bfloat16, 2e-2),
])
def test_decode_steps_match_oracle(dtype, state_dtype, tol):
    from rwkv_ops_b200 import Rwkv7DecodeState
    B, T, H = 3, 24, 5
    d = rwkv7_inputs(B, T, H, dtype=dtype, seed=77, with_state=True)
    o_ref, s_ref = _oracle(d, T)
    g = {n: d[n].cuda() for n in "rwkvab"}
    dec = Rwkv7DecodeState(B, H, state_dtype=state_dtype, initial_state=d["initial_state"].cuda())
    outs = [dec.step(*[g[n][:, t:t + 1] for n in "rwkvab"]) for t in range(T)]
    o = torch.cat(outs, dim=1)
    assert o.dtype == dtype and o.shape == (B, T, H, 64)
    assert rel_l2(o, o_ref) <= tol
    assert rel_l2(dec.final_state(), s_ref) <= tol


def test_decode_float32_equals_operator_bitwise():
    """float32 state: the in-place step is the T == 1 operator."""
    import rwkv_ops_b200 as ro
    B, T, H = 2, 6, 4
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=78, with_state=True, device="cuda")
    dec = ro.Rwkv7DecodeState(B, H, initial_state=d["initial_state"])
    s = d["initial_state"]
    for t in range(T):
        x = [d[n][:, t:t + 1] for n in "rwkvab"]
        o1 = dec.step(*x)
        o2, s = ro.generalized_delta_rule(*x, initial_state=s)
        assert torch.equal(o1, o2)
        assert torch.equal(dec.state, s)


def test_decode_broadcast_and_zero_state_and_3d_inputs():
    from rwkv_ops_b200 import Rwkv7DecodeState
    B, H = 4, 3
    d = rwkv7_inputs(B, 1, H, dtype=torch.float32, seed=79, device="cuda")
    s1 = 0.1 * torch.randn(1, H, 64, 64, device="cuda")
    a = Rwkv7DecodeState(B, H, initial_state=s1)
    b = Rwkv7DecodeState(B, H, initial_state=s1.expand(B, H, 64, 64))
    x4 = [d[n] for n in "rwkvab"]
    x3 = [t[:, 0] for t in x4]
    oa, ob = a.step(*x4), b.step(*x3)
    assert oa.shape == (B, 1, H, 64) and ob.shape == (B, H, 64)
    assert torch.equal(oa[:, 0], ob) and torch.equal(a.state, b.state)
    z = Rwkv7DecodeState(B, H)
    assert float(z.state.abs().max()) == 0.0
    z.step(*x4)
    assert float(z.state.abs().max()) > 0.0


def test_decode_steps_replay_from_a_cuda_graph():
    """A captured sequence of steps replays to the same outputs and state as eager execution."""
    from rwkv_ops_b200 import Rwkv7DecodeState
    B, T, H = 2, 8, 4
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=80, with_state=True, device="cuda")
    eager = Rwkv7DecodeState(B, H, initial_state=d["initial_state"])
    want = [eager.step(*[d[n][:, t:t + 1] for n in "rwkvab"]) for t in range(T)]
    dec = Rwkv7DecodeState(B, H, initial_state=d["initial_state"])
    static_in = {n: d[n].clone() for n in "rwkvab"}
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):      # warm-up outside the capture (loads the library)
        Rwkv7DecodeState(B, H).step(*[static_in[n][:, :1] for n in "rwkvab"])
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = [dec.step(*[static_in[n][:, t:t + 1] for n in "rwkvab"]) for t in range(T)]
    dec.state.copy_(d["initial_state"])   # the capture itself runs nothing
    graph.replay()
    torch.cuda.synchronize()
    for x, y in zip(got, want):
        assert torch.equal(x, y)
    assert torch.equal(dec.state, eager.state)


def test_decode_rejects_bad_arguments():
    from rwkv_ops_b200 import Rwkv7DecodeState
    with pytest.raises(ValueError):
        Rwkv7DecodeState(2, 2, state_dtype=torch.float16)
    dec = Rwkv7DecodeState(2, 2)
    x = torch.zeros(2, 2, 2, 64, device="cuda")
    with pytest.raises(ValueError):
        dec.step(x, x, x, x, x, x)


@pytest.mark.parametrize("state_dtype,tol_o,tol_s", [(torch.float32, 2e-2, 1e-4), (torch.bfloat16, 2e-2, 2e-2)])
def test_cfg3_full_shape_1024_chained_steps(state_dtype, tol_o, tol_s):
    """Benchmark configuration 3 at its own shape: B=256, H=64, bf16 tokens, 1024 consecutive steps with the
    state fed back (fresh token vectors every step).  Sampled (batch, head) units are checked against the
    oracle run over the unit's 1024-token sequence; the error after 1024 steps is the drift of the chain.
    The float32 state also goes through the T == 1 operator (rwkvb200_rwkv7_step) on a ping-pong pair."""
    import rwkv_ops_b200 as ro
    from oracle import generalized_delta_rule as oracle_gdr
    B, H, STEPS = 256, 64, 1024
    units = [(0, 0), (100, 37), (255, 63)]
    gen = torch.Generator(device="cuda").manual_seed(1003)
    s0 = 0.1 * torch.randn(B, H, 64, 64, device="cuda", generator=gen)
    dec = ro.Rwkv7DecodeState(B, H, state_dtype=state_dtype, initial_state=s0)
    s_op = s0.clone() if state_dtype == torch.float32 else None
    kept_in = {u: [] for u in units}
    kept_out = {u: [] for u in units}
    for t in range(STEPS):
        d = rwkv7_inputs(B, 1, H, dtype=torch.bfloat16, seed=5000 + t, device="cuda")
        x = [d[n] for n in "rwkvab"]
        o = dec.step(*x)
        if s_op is not None and t < 64:      # the operator path, bit for bit, over the first steps
            o2, s_op = ro.generalized_delta_rule(*x, initial_state=s_op)
            assert torch.equal(o, o2)
        for (b, h) in units:
            kept_in[(b, h)].append(torch.stack([t_[b, 0, h] for t_ in x]).cpu())
            kept_out[(b, h)].append(o[b, 0, h].cpu())
    if s_op is not None:
        pass
    final = dec.final_state()
    drift = {}
    for (b, h) in units:
        seq = torch.stack(kept_in[(b, h)], dim=1)            # [6, STEPS, 64]
        sub = [seq[i][None, :, None, :] for i in range(6)]
        o_ref, s_ref = oracle_gdr(*sub, initial_state=s0[b:b + 1, h:h + 1].cpu())
        o_got = torch.stack(kept_out[(b, h)])[None, :, None, :]
        drift[(b, h)] = (rel_l2(o_got, o_ref), rel_l2(o_got[:, -64:], o_ref[:, -64:]),
                         rel_l2(final[b:b + 1, h:h + 1], s_ref))
    print("cfg3 drift (o all steps, o last 64 steps, final state):", state_dtype, drift)
    for e_all, e_tail, e_s in drift.values():
        assert e_all < tol_o and e_tail < tol_o and e_s < tol_s
