"""Sequence-parallel RWKV7 delta rule: the sequence is split across ranks and chunk-boundary states
travel between neighbouring ranks by point-to-point messages (NCCL over NVLink on GPUs).

The reference has no multi-device support (``README.md:179``); this mode exists because the state
recurrence is a chain: rank ``g`` holds tokens ``[g*T/G, (g+1)*T/G)`` of every sequence, receives the
``[B, H, 64, 64]`` float32 state at its left boundary from rank ``g-1``, runs the ordinary operator on
its slice and sends its final state to rank ``g+1``.  The backward pass runs the same chain in reverse
with the gradient of the boundary state.  Splitting the batch into ``pipeline_groups`` groups lets rank
``g+1`` start on group ``j`` while rank ``g`` works on group ``j+1``, so the chain costs
``(G + groups - 1)`` group-steps instead of ``G * groups``.

Batch x head data parallelism needs none of this (units are independent); use this mode only when one
sequence is too long for one GPU.  Received states land in the receiver's own memory before any kernel
reads them; no kernel ever reads a peer's memory.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _default_local_op():
    from .rwkv7 import generalized_delta_rule
    return generalized_delta_rule


class _Chain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, h0, head_first, group, local_op, groups):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        prev_rank = ranks[rank - 1] if rank > 0 else None
        next_rank = ranks[rank + 1] if rank + 1 < world else None
        B = r.shape[0]
        H = r.shape[1] if head_first else r.shape[2]
        bounds = [(B * j) // groups for j in range(groups + 1)]
        outs, finals, graphs = [], [], []
        for j in range(groups):
            lo, hi = bounds[j], bounds[j + 1]
            if lo == hi:
                continue
            if prev_rank is not None:
                h_in = torch.empty(hi - lo, H, 64, 64, dtype=torch.float32, device=r.device)
                dist.recv(h_in, src=prev_rank, group=group)
            elif h0 is not None:
                h_in = (h0 if h0.shape[0] != 1 else h0.expand(B, -1, -1, -1))[lo:hi].contiguous()
            else:
                h_in = torch.zeros(hi - lo, H, 64, 64, dtype=torch.float32, device=r.device)
            with torch.enable_grad():
                leaves = [x[lo:hi].detach().requires_grad_(True) for x in (r, w, k, v, a, b)]
                h_leaf = h_in.detach().requires_grad_(True)
                o, ht = local_op(*leaves, initial_state=h_leaf, output_final_state=True, head_first=head_first)
            if next_rank is not None:
                dist.send(ht.detach().contiguous(), dst=next_rank, group=group)
            outs.append(o.detach())
            finals.append(ht.detach())
            graphs.append((lo, hi, leaves, h_leaf, o, ht))
        ctx.graphs, ctx.group = graphs, group
        ctx.prev_rank, ctx.next_rank = prev_rank, next_rank
        ctx.h0_shape = None if h0 is None else tuple(h0.shape)
        ctx.shape, ctx.dtype, ctx.device = tuple(r.shape), r.dtype, r.device
        return torch.cat(outs, 0), torch.cat(finals, 0)

    @staticmethod
    def backward(ctx, d_o, d_ht):
        grads = [torch.zeros(ctx.shape, dtype=ctx.dtype, device=ctx.device) for _ in range(6)]
        d_h0 = None
        if ctx.h0_shape is not None:
            d_h0 = torch.zeros((ctx.shape[0],) + ctx.h0_shape[1:], dtype=torch.float32, device=ctx.device)
        # same group order as the forward, so that neighbouring ranks overlap in the reverse chain too
        for lo, hi, leaves, h_leaf, o, ht in ctx.graphs:
            if ctx.next_rank is not None:
                d_state = torch.empty_like(ht)
                dist.recv(d_state, src=ctx.next_rank, group=ctx.group)
            elif d_ht is not None:
                d_state = d_ht[lo:hi].to(torch.float32)
            else:
                d_state = torch.zeros_like(ht)
            g_o = d_o[lo:hi] if d_o is not None else torch.zeros_like(o)
            res = torch.autograd.grad([o, ht], leaves + [h_leaf], [g_o.to(o.dtype), d_state], allow_unused=True)
            d_hin = res[6] if res[6] is not None else torch.zeros_like(h_leaf)
            if ctx.prev_rank is not None:
                dist.send(d_hin.contiguous(), dst=ctx.prev_rank, group=ctx.group)
            elif d_h0 is not None:
                d_h0[lo:hi] = d_hin
            for i in range(6):
                if res[i] is not None:
                    grads[i][lo:hi] = res[i]
        if d_h0 is not None and ctx.h0_shape[0] == 1:
            d_h0 = d_h0.sum(0, keepdim=True)
        return (*grads, d_h0, None, None, None, None)


def generalized_delta_rule_sp(r, w, k, v, a, b, initial_state: Optional[torch.Tensor] = None,
                              output_final_state: bool = True, head_first: bool = False,
                              group=None, pipeline_groups: int = 1, local_op: Optional[Callable] = None):
    """``generalized_delta_rule`` on a sequence split across the ranks of ``group`` (rank order =
    sequence order).  Every rank passes its own slice of the token tensors; ``initial_state`` is used on
    the first rank only.  Returns the local slice of ``o`` and, when ``output_final_state``, the state at
    the end of the local slice (the true final state on the last rank)."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    B = r.shape[0]
    groups = max(1, min(int(pipeline_groups), B))
    op = local_op or _default_local_op()
    o, ht = _Chain.apply(r, w, k, v, a, b, initial_state, bool(head_first), group, op, groups)
    return (o, ht) if output_final_state else o
