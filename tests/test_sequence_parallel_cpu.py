"""Control flow of the sequence-parallel mode on CPU ranks (gloo, world size 2 and 3): boundary states
and their gradients hop between ranks in the right order, with and without batch pipelining.  The local
operator is the CPU oracle, so no GPU is involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import generalized_delta_rule as oracle_gdr
from rwkv_ops_b200.sequence_parallel import generalized_delta_rule_sp
from rwkv_ops_b200.workloads import rwkv7_inputs, rel_l2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, groups, with_state, out, mid_loss=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    B, T, H = 3, 12 * world, 2
    d = rwkv7_inputs(B, T, H, seed=42, with_state=with_state, with_grads=True)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    loc = {n: d[n][:, sl].clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True) if with_state else None
    o, s = generalized_delta_rule_sp(*[loc[n] for n in "rwkvab"], initial_state=h0 if rank == 0 else None,
                                     pipeline_groups=groups, local_op=oracle_gdr)
    loss = (o * d["d_out"][:, sl]).sum()
    if rank == world - 1:
        loss = loss + (s * d["d_state"]).sum()
    elif mid_loss:      # a loss on the boundary state of a rank that is not the last one
        loss = loss + (s * (0.5 + rank) * d["d_state"]).sum()
    loss.backward()
    res = {"o": o.detach(), "s": s.detach(), **{f"d{n}": loc[n].grad for n in "rwkvab"}}
    if with_state and rank == 0:
        res["dh0"] = h0.grad
    torch.save(res, os.path.join(out, f"rank{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,groups,with_state", [(2, 1, True), (2, 3, False), (3, 2, True)])
def test_chain_matches_single_process(tmp_path, world, groups, with_state):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, groups, with_state, str(tmp_path)), nprocs=world, join=True)
    B, T, H = 3, 12 * world, 2
    d = rwkv7_inputs(B, T, H, seed=42, with_state=with_state, with_grads=True)
    full = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True) if with_state else None
    o, s = oracle_gdr(*[full[n] for n in "rwkvab"], initial_state=h0)
    ((o * d["d_out"]).sum() + (s * d["d_state"]).sum()).backward()
    for rank in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"rank{rank}.pt"))
        sl = slice(rank * T // world, (rank + 1) * T // world)
        assert rel_l2(res["o"], o[:, sl]) < 1e-5
        for n in "rwkvab":
            assert rel_l2(res[f"d{n}"], full[n].grad[:, sl]) < 1e-4, (rank, n)
        if rank == world - 1:
            assert rel_l2(res["s"], s) < 1e-5
        if with_state and rank == 0:
            assert rel_l2(res["dh0"], h0.grad) < 1e-4


def test_loss_on_an_inner_boundary_state_is_differentiated(tmp_path):
    """The state a rank returns is the state at the end of its slice; a loss on it (on a rank that is not the
    last) must reach every token before that boundary, on this rank and on the ranks to its left."""
    world = 3
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 1, True, str(tmp_path), True), nprocs=world, join=True)
    B, T, H = 3, 12 * world, 2
    d = rwkv7_inputs(B, T, H, seed=42, with_state=True, with_grads=True)
    full = {n: d[n].clone().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].clone().requires_grad_(True)
    o, s = oracle_gdr(*[full[n] for n in "rwkvab"], initial_state=h0)
    loss = (o * d["d_out"]).sum() + (s * d["d_state"]).sum()
    for rank in range(world - 1):
        end = (rank + 1) * T // world
        _, s_mid = oracle_gdr(*[full[n][:, :end] for n in "rwkvab"], initial_state=h0)
        loss = loss + (s_mid * (0.5 + rank) * d["d_state"]).sum()
    loss.backward()
    for rank in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"rank{rank}.pt"))
        sl = slice(rank * T // world, (rank + 1) * T // world)
        for n in "rwkvab":
            assert rel_l2(res[f"d{n}"], full[n].grad[:, sl]) < 1e-4, (rank, n)
    assert rel_l2(torch.load(os.path.join(str(tmp_path), "rank0.pt"))["dh0"], h0.grad) < 1e-4
