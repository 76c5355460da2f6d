"""Device-timed micro-benchmarks of the individual operators (CUDA events, inputs resident in HBM).

    python microbench.py step  [--B 256 --H 64 --steps 50 --dtype bf16]
    python microbench.py step  --state-dtype bf16      (in place, bfloat16 state)
    python microbench.py wkv6  [--B 16 --T 4096 --H 32 --steps 5]
    python microbench.py rwkv7 [--B 8 --T 4096 --H 32 --steps 5 --dtype bf16 --algo auto]
    python microbench.py varlen [--B 8 --T 4096 --H 32]     (packed sequences vs padded)
    python microbench.py fused  [--B 8 --T 4096 --H 32]     (producers of w, a, b fused in vs torch)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 microbench.py sp

Each prints one JSON line with the time per call and the achieved algorithmic bandwidth; small cases of
these commands are what the profiler captures.
"""
from __future__ import annotations

import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import rwkv_ops_b200 as ro
from rwkv_ops_b200 import _lib
from rwkv_ops_b200.workloads import rwkv7_inputs, wkv6_inputs

DT = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}


def _time(fn, steps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _lib.profile(True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    prof = _lib.profile_results()
    _lib.profile(False)
    return e0.elapsed_time(e1) / steps, {k: v[0] / max(v[1], 1) for k, v in prof.items()}


def bench_step(a):
    """Configuration 3: T=1 decode, fp32 state [B,H,64,64] fed back step after step."""
    dt = DT[a.dtype]
    n_in = 8   # distinct input sets so consecutive steps do not reuse L2-resident token vectors
    ds = [rwkv7_inputs(a.B, 1, a.H, dtype=dt, seed=1003 + i, device="cuda") for i in range(n_in)]
    state = 0.1 * torch.randn(a.B, a.H, 64, 64, device="cuda")
    lib = _lib.load()
    code = _lib.dtype_code(dt)
    o = torch.empty(a.B, a.H, 64, dtype=dt, device="cuda")
    bufs = [state, torch.empty_like(state)]
    i = [0]

    def fn():
        d = ds[i[0] % n_in]
        src, dst = bufs[i[0] & 1], bufs[(i[0] + 1) & 1]
        rc = lib.rwkvb200_rwkv7_step(*[d[n].data_ptr() for n in "rwkvab"], src.data_ptr(), a.B, dst.data_ptr(),
                                     o.data_ptr(), a.B, a.H, 64, code, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        i[0] += 1

    es = torch.finfo(dt).bits // 8
    if a.state_dtype:      # in place on one state buffer (float32 or bfloat16)
        sdt = DT[a.state_dtype]
        inplace = state.to(sdt)
        scode = _lib.dtype_code(sdt)
        ss = torch.finfo(sdt).bits // 8

        def fn():   # noqa: F811
            d = ds[i[0] % n_in]
            rc = lib.rwkvb200_rwkv7_decode_step(*[d[n].data_ptr() for n in "rwkvab"], inplace.data_ptr(), scode,
                                                o.data_ptr(), a.B, a.H, 64, code,
                                                torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            i[0] += 1

        ms, kern = _time(fn, a.steps)
        nbytes = a.B * a.H * (2 * 64 * 64 * ss + 7 * 64 * es)
        return {"op": "rwkv7_decode_step", "B": a.B, "H": a.H, "dtype": a.dtype, "state_dtype": a.state_dtype,
                "us_per_step": 1e3 * ms, "algorithmic_bytes": nbytes, "GBps": nbytes / (ms / 1e3) / 1e9,
                "state_bytes_vs_l2": "state updated in place, %.0f MB against the 126 MB L2" % (a.B * a.H * 4096 * ss / 1e6),
                "kernel_ms": kern}
    ms, kern = _time(fn, a.steps)
    nbytes = a.B * a.H * (2 * 64 * 64 * 4 + 7 * 64 * es)
    return {"op": "rwkv7_step", "B": a.B, "H": a.H, "dtype": a.dtype, "us_per_step": 1e3 * ms,
            "algorithmic_bytes": nbytes, "GBps": nbytes / (ms / 1e3) / 1e9,
            "state_bytes_vs_l2": "state ping-pong buffers (2 x %.0f MB) exceed the 126 MB L2" % (a.B * a.H * 16384 / 1e6),
            "kernel_ms": kern}


def bench_varlen(a):
    """Packed variable-length batch (lengths uniform in [T/16, T], seeded) against the same sequences padded
    to T with the reference's recipe (w = -1e9 on the padding), forward + backward, bf16."""
    from rwkv_ops_b200 import generalized_delta_rule_varlen
    gen = torch.Generator().manual_seed(1001)
    n_seq = a.B
    if a.tail:      # the padding pattern of benchmark configuration 2: T minus up to `tail` tokens
        lens = (a.T - torch.randint(0, a.tail + 1, (n_seq,), generator=gen)).tolist()
    else:
        lens = torch.randint(a.T // 16, a.T + 1, (n_seq,), generator=gen).tolist()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    total = cu[-1]
    d = rwkv7_inputs(1, total, a.H, dtype=torch.bfloat16, seed=1001, device="cuda", with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    cu_t = ro.PackedSequences(cu, "cuda")      # prepared once, as for all the layers of a step
    d_state = 0.1 * torch.randn(n_seq, a.H, 64, 64, device="cuda")

    def packed():
        for t in g.values():      # no accumulation into .grad of an earlier step
            t.grad = None
        o, s = generalized_delta_rule_varlen(*[g[n] for n in "rwkvab"], cu_t)
        torch.autograd.backward([o, s], [d["d_out"], d_state])

    pad = {n: torch.zeros(n_seq, a.T, a.H, 64, dtype=torch.bfloat16, device="cuda") for n in "rwkvab"}
    pad["w"].fill_(-1e9)
    for i, n_tok in enumerate(lens):
        for n in "rwkvab":
            pad[n][i, :n_tok] = d[n][0, cu[i]:cu[i + 1]].detach()
    gp = {n: pad[n].requires_grad_(True) for n in "rwkvab"}
    d_out_pad = torch.randn(n_seq, a.T, a.H, 64, device="cuda").bfloat16()

    def padded():
        for t in gp.values():
            t.grad = None
        o, s = ro.generalized_delta_rule(*[gp[n] for n in "rwkvab"])
        torch.autograd.backward([o, s], [d_out_pad, d_state])

    ms_packed, kern = _time(packed, a.steps)
    ms_padded, _ = _time(padded, a.steps)
    return {"op": "rwkv7_fwd_bwd_varlen", "n_seq": n_seq, "max_len": a.T, "H": a.H, "tokens": total,
            "padded_tokens": n_seq * a.T, "ms_packed": ms_packed, "ms_padded": ms_padded,
            "tokens_per_s_packed": total / (ms_packed / 1e3), "tokens_per_s_padded": total / (ms_padded / 1e3),
            "kernel_ms": kern}


def bench_fused(a):
    """Forward + backward with the producers of w, a, b inside the operator, against the same producers as
    torch elementwise ops (with autograd) in front of the plain operator; bf16."""
    from rwkv_ops_b200.fused import producers
    gen = torch.Generator(device="cuda").manual_seed(1001)
    names = ("r", "w_pre", "k", "v", "kk_pre", "a_pre")
    x = {n: torch.randn(a.B, a.T, a.H, 64, generator=gen, device="cuda").bfloat16().requires_grad_(True) for n in names}
    d_out = torch.randn(a.B, a.T, a.H, 64, generator=gen, device="cuda").bfloat16()
    d_state = 0.1 * torch.randn(a.B, a.H, 64, 64, generator=gen, device="cuda")

    def clear():      # no accumulation into .grad of an earlier step (six more passes over the tensors)
        for t in x.values():
            t.grad = None

    def fused():
        clear()
        o, s = ro.generalized_delta_rule_fused(*[x[n] for n in names])
        torch.autograd.backward([o, s], [d_out, d_state])

    def unfused():
        clear()
        w, aa, bb = producers(x["w_pre"], x["kk_pre"], x["a_pre"])
        o, s = ro.generalized_delta_rule(x["r"], w, x["k"], x["v"], aa, bb)
        torch.autograd.backward([o, s], [d_out, d_state])

    ms_fused, kern = _time(fused, a.steps)
    ms_unfused, _ = _time(unfused, a.steps)
    return {"op": "rwkv7_fwd_bwd_fused_producers", "B": a.B, "T": a.T, "H": a.H, "ms_fused": ms_fused,
            "ms_unfused_torch_producers": ms_unfused, "tokens_per_s_fused": a.B * a.T / (ms_fused / 1e3),
            "tokens_per_s_unfused": a.B * a.T / (ms_unfused / 1e3), "kernel_ms": kern}


def bench_sp(a):
    """Sequence-parallel forward + backward: every rank holds T tokens of each of B sequences (the whole
    sequence is world x T long); run under torchrun, one rank per GPU.  Time = max over ranks."""
    import torch.distributed as dist
    from rwkv_ops_b200.sequence_parallel import generalized_delta_rule_sp
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    d = rwkv7_inputs(a.B, a.T, a.H, dtype=torch.bfloat16, seed=1001 + rank, device="cuda", with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}

    def step():
        for t in g.values():      # no accumulation into .grad of an earlier step
            t.grad = None
        o, s = generalized_delta_rule_sp(*[g[n] for n in "rwkvab"], pipeline_groups=a.groups)
        torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    res = {"op": "rwkv7_fwd_bwd_sequence_parallel", "ranks": world, "B": a.B, "tokens_per_rank": a.T,
           "sequence_length": world * a.T, "H": a.H, "pipeline_groups": a.groups, "ms_per_step": float(ms),
           "tokens_per_s": a.B * a.T * world / (float(ms) / 1e3)}
    dist.destroy_process_group()
    return res if rank == 0 else None


def bench_wkv6(a):
    """Configuration 4: wkv6 forward + backward, fp32, 4 initial states and a state_map."""
    dt = DT[a.dtype]
    d = wkv6_inputs(a.B, a.T, a.H, dtype=dt, seed=1004, device="cuda", n_state=4, with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].requires_grad_(True)
    op = ro.RWKV6_OP(64, a.T)

    def fn():
        y, s = op(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0, state_map=d["state_map"])
        torch.autograd.backward([y, s], [d["d_y"], d["d_state"]])
        for t in list(g.values()) + [s0]:
            t.grad = None

    ms, kern = _time(fn, a.steps)
    es = torch.finfo(dt).bits // 8
    nbytes = a.B * a.T * a.H * 64 * es * 14
    return {"op": "wkv6_fwd_bwd", "B": a.B, "T": a.T, "H": a.H, "dtype": a.dtype, "ms_per_step": ms,
            "tokens_per_s": a.B * a.T / (ms / 1e3), "algorithmic_bytes": nbytes,
            "GBps": nbytes / (ms / 1e3) / 1e9, "kernel_ms": kern}


def bench_rwkv7(a):
    dt = DT[a.dtype]
    os.environ["RWKV_OPS_B200_RWKV7_ALGO"] = a.algo
    d = rwkv7_inputs(a.B, a.T, a.H, dtype=dt, seed=1001, device="cuda", with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}

    def fn():
        o, s = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"])
        if not a.fwd_only:
            torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])
            for t in g.values():
                t.grad = None

    ms, kern = _time(fn, a.steps)
    es = torch.finfo(dt).bits // 8
    nbytes = a.B * a.T * a.H * 64 * es * (7 if a.fwd_only else 20)
    return {"op": "rwkv7_fwd" if a.fwd_only else "rwkv7_fwd_bwd", "algo": a.algo, "B": a.B, "T": a.T, "H": a.H,
            "dtype": a.dtype, "ms_per_step": ms, "tokens_per_s": a.B * a.T / (ms / 1e3),
            "algorithmic_bytes": nbytes, "GBps": nbytes / (ms / 1e3) / 1e9, "kernel_ms": kern}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["step", "wkv6", "rwkv7", "varlen", "sp", "fused"])
    ap.add_argument("--tail", type=int, default=0,
                    help="varlen: lengths are T minus a random 0..tail tokens instead of uniform in [T/16, T]")
    ap.add_argument("--groups", type=int, default=4, help="sp: batch groups pipelined along the chain of ranks")
    ap.add_argument("--B", type=int)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--H", type=int)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--dtype", default=None)
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--state-dtype", default=None, choices=["f32", "bf16"],
                    help="step: decode in place on one state buffer of this type (rwkvb200_rwkv7_decode_step)")
    ap.add_argument("--fwd-only", action="store_true")
    a = ap.parse_args()
    defaults = {"step": (256, 64, "bf16"), "wkv6": (16, 32, "f32"), "rwkv7": (8, 32, "bf16"), "varlen": (8, 32, "bf16"), "sp": (8, 32, "bf16"), "fused": (8, 32, "bf16")}[a.op]
    a.B = a.B or defaults[0]
    a.H = a.H or defaults[1]
    a.dtype = a.dtype or defaults[2]
    if a.op != "sp":
        torch.cuda.set_device(0)
    res = {"step": bench_step, "wkv6": bench_wkv6, "rwkv7": bench_rwkv7, "varlen": bench_varlen, "sp": bench_sp, "fused": bench_fused}[a.op](a)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
