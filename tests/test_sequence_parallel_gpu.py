"""Sequence-parallel mode on real GPUs.  The phases of the local operator (state-independent work, scans,
token gradients) are checked on one GPU against the whole call and the oracle; the two-rank run (NCCL
point-to-point, each rank with half of every sequence) is checked against the CPU oracle run over the whole
sequence, and is skipped on a single-GPU box."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkv_ops_b200.workloads import rwkv7_inputs, rel_l2

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rwkv_ops_b200.sequence_parallel import generalized_delta_rule_sp
    B, T, H = 4, 512, 4
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=43, with_state=True, with_grads=True)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    loc = {n: d[n][:, sl].cuda().contiguous().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = generalized_delta_rule_sp(*[loc[n] for n in "rwkvab"], initial_state=h0 if rank == 0 else None,
                                     pipeline_groups=2)
    grads = [d["d_out"][:, sl].cuda().contiguous(), d["d_state"].cuda() if rank == world - 1 else torch.zeros_like(s)]
    torch.autograd.backward([o, s], grads)
    torch.cuda.synchronize()
    res = {"o": o.detach().cpu(), "s": s.detach().cpu(), **{f"d{n}": loc[n].grad.cpu() for n in "rwkvab"}}
    if rank == 0:
        res["dh0"] = h0.grad.cpu()
    torch.save(res, os.path.join(out, f"rank{rank}.pt"))
    dist.destroy_process_group()


def _oracle_full(B, T, H):
    from oracle import generalized_delta_rule as oracle_gdr
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=43, with_state=True, with_grads=True)
    full = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True)
    o, s = oracle_gdr(*[full[n] for n in "rwkvab"], initial_state=h0)
    ((o * d["d_out"].float()).sum() + (s * d["d_state"]).sum()).backward()
    return d, full, h0, o, s


def test_two_gpu_chain_matches_the_oracle(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s_ = socket.socket(); s_.bind(("127.0.0.1", 0)); port = s_.getsockname()[1]; s_.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    B, T, H = 4, 512, 4
    d, full, h0, o, s = _oracle_full(B, T, H)
    for rank in range(2):
        res = torch.load(os.path.join(str(tmp_path), f"rank{rank}.pt"))
        sl = slice(rank * T // 2, (rank + 1) * T // 2)
        assert rel_l2(res["o"], o[:, sl]) < 2e-2
        for n in "rwkvab":
            assert rel_l2(res[f"d{n}"], full[n].grad[:, sl]) < 2e-2, (rank, n)
    assert rel_l2(res["s"], s) < 2e-2
    assert rel_l2(torch.load(os.path.join(str(tmp_path), "rank0.pt"))["dh0"], h0.grad) < 2e-2


def test_phases_on_one_gpu_chain_two_halves():
    """The phased operator on one GPU, playing both ranks of a two-way split in the order a real run
    interleaves them (both `prepare` phases first, then the scans left to right; backward: both `prepare`
    phases, the reverse scans right to left, then both `finish` phases), against the oracle run over the
    whole sequence; and the phases of one slice against the unsplit call, bit for bit."""
    import rwkv_ops_b200 as ro
    from rwkv_ops_b200.sequence_parallel import ChunkedPhasedOp
    B, T, H = 4, 512, 4
    d, full, h0, o_ref, s_ref = _oracle_full(B, T, H)
    op = ChunkedPhasedOp()
    half = T // 2
    tok = [[d[n][:, i * half:(i + 1) * half].cuda().contiguous() for n in "rwkvab"] for i in range(2)]
    st = [op.prepare_fwd(*tok[i], False) for i in range(2)]
    o0, h_mid = op.scan_fwd(st[0], d["initial_state"].cuda())
    o1, h_end = op.scan_fwd(st[1], h_mid)
    assert rel_l2(torch.cat([o0, o1], 1), o_ref) < 2e-2 and rel_l2(h_end, s_ref) < 2e-2
    for i in range(2):
        op.prepare_bwd(st[i], d["d_out"][:, i * half:(i + 1) * half].cuda())
    d_mid = op.scan_bwd(st[1], d["d_state"].cuda()).clone()
    d_h0 = op.scan_bwd(st[0], d_mid).clone()
    grads = [op.finish_bwd(st[i]) for i in range(2)]
    for j, n in enumerate("rwkvab"):
        got = torch.cat([grads[0][j], grads[1][j]], 1)
        assert rel_l2(got, full[n].grad) < 2e-2, n
    assert rel_l2(d_h0, h0.grad) < 2e-2
    # one slice, phase by phase, equals the unsplit operator call on that slice
    g = {n: t.clone().requires_grad_(True) for n, t in zip("rwkvab", tok[1])}
    hm = h_mid.clone().requires_grad_(True)
    o_w, s_w = ro.generalized_delta_rule(*[g[n] for n in "rwkvab"], initial_state=hm)
    torch.autograd.backward([o_w, s_w], [d["d_out"][:, half:].cuda(), d["d_state"].cuda()])
    assert torch.equal(o_w, o1) and torch.equal(s_w, h_end)
    for j, n in enumerate("rwkvab"):
        assert torch.equal(g[n].grad, grads[1][j]), n
    assert torch.equal(hm.grad, d_mid)
    torch.cuda.synchronize()
    from rwkv_ops_b200 import _lib
    assert _lib.load().rwkvb200_device_status(1) == 0


def test_phases_with_a_unit_beyond_the_decay_range():
    """One head of the right half decays faster than the tensor-core kernels' range: its outputs and gradients
    come from the recurrence, and so must its share of the state gradient that the right rank hands to the left
    one after its scan phase (before its token gradients exist)."""
    from oracle import generalized_delta_rule as oracle_gdr
    from rwkv_ops_b200.sequence_parallel import ChunkedPhasedOp
    B, T, H = 2, 256, 3
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=47, with_state=True, with_grads=True)
    w = d["w"].float()
    w[1, T // 2:, 2] = 1.0      # exp(1) = 2.7 per token: 87 over half a chunk, beyond the limit of 60
    d["w"] = w.bfloat16()
    full = {n: d[n].float().clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True)
    o_ref, s_ref = oracle_gdr(*[full[n] for n in "rwkvab"], initial_state=h0)
    ((o_ref * d["d_out"].float()).sum() + (s_ref * d["d_state"]).sum()).backward()
    op = ChunkedPhasedOp()
    half = T // 2
    tok = [[d[n][:, i * half:(i + 1) * half].cuda().contiguous() for n in "rwkvab"] for i in range(2)]
    st = [op.prepare_fwd(*tok[i], False) for i in range(2)]
    o0, h_mid = op.scan_fwd(st[0], d["initial_state"].cuda())
    o1, h_end = op.scan_fwd(st[1], h_mid)
    assert rel_l2(torch.cat([o0, o1], 1), o_ref) < 2e-2 and rel_l2(h_end, s_ref) < 2e-2
    for i in range(2):
        op.prepare_bwd(st[i], d["d_out"][:, i * half:(i + 1) * half].cuda())
    d_mid = op.scan_bwd(st[1], d["d_state"].cuda()).clone()
    d_h0 = op.scan_bwd(st[0], d_mid).clone()
    grads = [op.finish_bwd(st[i]) for i in range(2)]
    for j, n in enumerate("rwkvab"):
        got = torch.cat([grads[0][j], grads[1][j]], 1)
        assert torch.isfinite(got.float()).all(), n
        assert rel_l2(got, full[n].grad) < 2e-2, n
        # the left half alone: it sees the marked unit only through d_mid
        assert rel_l2(grads[0][j][1, :, 2], full[n].grad[1, :half, 2]) < 2e-2, n
    assert rel_l2(d_h0, h0.grad) < 2e-2
