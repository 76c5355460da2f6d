"""Sequence-parallel mode on real GPUs (NCCL point-to-point): two ranks, each with half of every
sequence, against one GPU running the whole sequence.  Skipped on a single-GPU box."""
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


def test_two_gpu_chain_matches_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import rwkv_ops_b200 as ro
    s_ = socket.socket(); s_.bind(("127.0.0.1", 0)); port = s_.getsockname()[1]; s_.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    B, T, H = 4, 512, 4
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=43, with_state=True, with_grads=True)
    full = {n: d[n].cuda().requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].cuda().requires_grad_(True)
    o, s = ro.generalized_delta_rule(*[full[n] for n in "rwkvab"], initial_state=h0)
    torch.autograd.backward([o, s], [d["d_out"].cuda(), d["d_state"].cuda()])
    for rank in range(2):
        res = torch.load(os.path.join(str(tmp_path), f"rank{rank}.pt"))
        sl = slice(rank * T // 2, (rank + 1) * T // 2)
        assert rel_l2(res["o"], o[:, sl]) < 2e-2
        for n in "rwkvab":
            assert rel_l2(res[f"d{n}"], full[n].grad[:, sl]) < 2e-2, (rank, n)
    assert rel_l2(res["s"], s) < 2e-2
    assert rel_l2(torch.load(os.path.join(str(tmp_path), "rank0.pt"))["dh0"], h0.grad) < 2e-2
