"""Sequence-parallel RWKV7 delta rule: the sequence is split across ranks and chunk-boundary states
travel between neighbouring ranks by point-to-point messages (NCCL over NVLink on GPUs).

The reference has no multi-device support (``README.md:179``).  The state recurrence is a chain: rank ``g``
holds tokens ``[g*T/G, (g+1)*T/G)`` of every sequence and needs the ``[B, H, 64, 64]`` float32 state at its
left boundary from rank ``g-1``.  What keeps the chain short is that most of the operator does not depend on
that state.  The work of a rank is split into phases:

* forward: ``prepare`` (everything inside the chunks: decay prefix sums, the four A matrices, the triangular
  inverse; about three quarters of the forward) runs on all ranks at once; only ``scan`` (the state walking
  through the chunks) waits for the left neighbour's final state and hands its own to the right neighbour;
* backward: ``prepare`` and ``finish`` (all token gradients) run on all ranks at once; only the reverse scan
  waits for the gradient of the state from the right neighbour.

With ``G`` ranks a step therefore costs about ``(prepare + finish) / G + scans`` instead of the whole operator
once per rank in turn.  The phased operator is the chunked tensor-core path (bfloat16 tokens), driven through
the phase flags of ``rwkvb200_rwkv7_fwd`` / ``_bwd``; any other local operator (float32 tokens, or the CPU
oracle in the control-flow tests) runs as a plain chain, optionally pipelined over ``pipeline_groups`` groups
of batch rows.

Batch x head data parallelism needs none of this (units are independent); use this mode when one sequence is
too long for one GPU.  Received states land in the receiver's own memory before any kernel reads them; no
kernel ever reads a peer's memory.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _default_local_op():
    from .rwkv7 import generalized_delta_rule
    return generalized_delta_rule


class PhasedLocalOp:
    """Interface of a local operator whose state-independent work can run ahead of the chain.

    ``prepare_fwd(r, w, k, v, a, b, head_first) -> st``; ``scan_fwd(st, h_in, o_out, ht_out) -> (o, ht)``;
    ``prepare_bwd(st, d_o, grads_out)``; ``scan_bwd(st, d_ht) -> d_h_in``; ``finish_bwd(st) -> six token
    gradients``.  ``o_out``, ``ht_out`` and the six ``grads_out`` are views (one group of batch rows) of the
    caller's full-size results: an operator that can write its results in place does, so that nothing is
    copied afterwards.
    """


class ChunkedPhasedOp(PhasedLocalOp):
    """The chunked tensor-core operator (bfloat16 token tensors on a CUDA device), one C-ABI call per phase."""

    class _St:
        pass

    def prepare_fwd(self, r, w, k, v, a, b, head_first):
        from . import _lib
        lib = _lib.load()
        dev = _lib.require_cuda(r, w, k, v, a, b)
        st = self._St()
        st.tok = [x.to(torch.bfloat16).contiguous() for x in (r, w, k, v, a, b)]
        st.head_first = bool(head_first)
        if head_first:
            st.B, st.H, st.T, K = r.shape
        else:
            st.B, st.T, st.H, K = r.shape
        if K != 64:
            raise ValueError("head size must be 64")
        st.dev = dev
        st.algo = _lib.ALGO_CHUNKED | _lib.ALGO_KEEP
        with torch.cuda.device(dev):
            st.nws = lib.rwkvb200_rwkv7_fwd_workspace_bytes(st.B, st.T, st.H, 64, _lib.BF16, st.algo)
            st.ws = torch.empty(st.nws, dtype=torch.uint8, device=dev)
            rc = lib.rwkvb200_rwkv7_fwd(*[t.data_ptr() for t in st.tok], None, 0, None, None, st.ws.data_ptr(),
                                        st.nws, st.B, st.T, st.H, 64, _lib.BF16, int(st.head_first),
                                        st.algo | _lib.PHASE_PREPARE, _lib.stream_ptr(dev))
            _lib.check(rc, "rwkv7_fwd (prepare)")
        return st

    @staticmethod
    def _usable(x, like):
        return (x is not None and x.is_contiguous() and x.dtype == like.dtype and x.shape == like.shape
                and x.device == like.device)

    def scan_fwd(self, st, h_in, o_out=None, ht_out=None):
        from . import _lib
        lib = _lib.load()
        st.h_in = None if h_in is None else h_in.to(torch.float32).contiguous()
        o = o_out if self._usable(o_out, st.tok[0]) else torch.empty_like(st.tok[0])
        ht = torch.empty(st.B, st.H, 64, 64, dtype=torch.float32, device=st.dev)
        if ht_out is not None and ht_out.is_contiguous() and ht_out.dtype == ht.dtype and ht_out.shape == ht.shape:
            ht = ht_out
        with torch.cuda.device(st.dev):
            rc = lib.rwkvb200_rwkv7_fwd(*[t.data_ptr() for t in st.tok], _lib.ptr(st.h_in),
                                        0 if st.h_in is None else st.h_in.shape[0], o.data_ptr(), ht.data_ptr(),
                                        st.ws.data_ptr(), st.nws, st.B, st.T, st.H, 64, _lib.BF16,
                                        int(st.head_first), st.algo | _lib.PHASE_SCAN, _lib.stream_ptr(st.dev))
            _lib.check(rc, "rwkv7_fwd (scan)")
        return o, ht

    def _bwd(self, st, phase, what):
        from . import _lib
        lib = _lib.load()
        with torch.cuda.device(st.dev):
            rc = lib.rwkvb200_rwkv7_bwd(*[t.data_ptr() for t in st.tok], _lib.ptr(st.h_in),
                                        0 if st.h_in is None else st.h_in.shape[0], st.d_o.data_ptr(),
                                        _lib.ptr(st.d_ht), *[g.data_ptr() for g in st.grads], st.d_h0.data_ptr(),
                                        st.ws.data_ptr(), st.nws, st.B, st.T, st.H, 64, _lib.BF16,
                                        int(st.head_first), st.algo | phase, _lib.stream_ptr(st.dev))
            _lib.check(rc, f"rwkv7_bwd ({what})")

    def prepare_bwd(self, st, d_o, grads_out=None):
        from . import _lib
        st.d_o = d_o.to(torch.bfloat16).contiguous()
        st.d_ht = None
        if grads_out is not None and all(self._usable(g, st.tok[0]) for g in grads_out):
            st.grads = list(grads_out)
        else:
            st.grads = [torch.empty_like(st.tok[0]) for _ in range(6)]
        st.d_h0 = torch.empty(st.B, st.H, 64, 64, dtype=torch.float32, device=st.dev)
        self._bwd(st, _lib.PHASE_PREPARE, "prepare")

    def scan_bwd(self, st, d_ht):
        from . import _lib
        st.d_ht = None if d_ht is None else d_ht.to(torch.float32).contiguous()
        self._bwd(st, _lib.PHASE_SCAN, "scan")
        return st.d_h0

    def finish_bwd(self, st):
        from . import _lib
        self._bwd(st, _lib.PHASE_FINISH, "finish")
        return st.grads


class ChainPhasedOp(PhasedLocalOp):
    """Any ``generalized_delta_rule``-like callable behind the phased interface (all work in the scans):
    the plain chain, used for float32 tokens and, with the CPU oracle, by the control-flow tests."""

    class _St:
        pass

    def __init__(self, local_op: Callable):
        self.local_op = local_op

    def prepare_fwd(self, r, w, k, v, a, b, head_first):
        st = self._St()
        st.head_first = bool(head_first)
        st.leaves = [x.detach().requires_grad_(True) for x in (r, w, k, v, a, b)]
        return st

    def scan_fwd(self, st, h_in, o_out=None, ht_out=None):
        B = st.leaves[0].shape[0]
        H = st.leaves[0].shape[1] if st.head_first else st.leaves[0].shape[2]
        if h_in is None:
            h_in = torch.zeros(B, H, 64, 64, dtype=torch.float32, device=st.leaves[0].device)
        with torch.enable_grad():
            st.h_leaf = h_in.detach().requires_grad_(True)
            st.o, st.ht = self.local_op(*st.leaves, initial_state=st.h_leaf, output_final_state=True,
                                        head_first=st.head_first)
        return st.o.detach(), st.ht.detach()

    def prepare_bwd(self, st, d_o, grads_out=None):
        st.d_o = d_o

    def scan_bwd(self, st, d_ht):
        if d_ht is None:
            d_ht = torch.zeros_like(st.ht)
        res = torch.autograd.grad([st.o, st.ht], st.leaves + [st.h_leaf], [st.d_o.to(st.o.dtype), d_ht],
                                  allow_unused=True)
        st.res = [g if g is not None else torch.zeros_like(x) for g, x in zip(res, st.leaves + [st.h_leaf])]
        return st.res[6]

    def finish_bwd(self, st):
        return st.res[:6]


class _Chain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, h0, head_first, group, op, groups):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        prev_rank = ranks[rank - 1] if rank > 0 else None
        next_rank = ranks[rank + 1] if rank + 1 < world else None
        B = r.shape[0]
        H = r.shape[1] if head_first else r.shape[2]
        bounds = [(B * j) // groups for j in range(groups + 1)]
        spans = [(bounds[j], bounds[j + 1]) for j in range(groups) if bounds[j] < bounds[j + 1]]
        # everything that does not wait for a neighbour first: it runs while the left ranks scan
        states = [op.prepare_fwd(*(x[lo:hi] for x in (r, w, k, v, a, b)), head_first) for lo, hi in spans]
        # full-size results; every group writes its rows in place where the operator can
        o_full = torch.empty_like(r)
        ht_full = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device)
        for (lo, hi), st in zip(spans, states):
            if prev_rank is not None:
                h_in = torch.empty(hi - lo, H, 64, 64, dtype=torch.float32, device=r.device)
                dist.recv(h_in, src=prev_rank, group=group)
            elif h0 is not None:
                h_in = (h0 if h0.shape[0] != 1 else h0.expand(B, -1, -1, -1))[lo:hi].contiguous()
            else:
                h_in = None
            o, ht = op.scan_fwd(st, h_in, o_full[lo:hi], ht_full[lo:hi])
            if next_rank is not None:
                dist.send(ht.contiguous(), dst=next_rank, group=group)
            if o.data_ptr() != o_full[lo:hi].data_ptr():
                o_full[lo:hi] = o
            if ht.data_ptr() != ht_full[lo:hi].data_ptr():
                ht_full[lo:hi] = ht
        ctx.op, ctx.states, ctx.spans, ctx.group = op, states, spans, group
        ctx.prev_rank, ctx.next_rank = prev_rank, next_rank
        ctx.h0_shape = None if h0 is None else tuple(h0.shape)
        ctx.shape, ctx.dtype, ctx.device = tuple(r.shape), r.dtype, r.device
        ctx.state_tail = (H, 64, 64)
        ctx.set_materialize_grads(False)
        return o_full, ht_full

    @staticmethod
    def backward(ctx, d_o, d_ht):
        op = ctx.op
        grads = [torch.empty(ctx.shape, dtype=ctx.dtype, device=ctx.device) for _ in range(6)]
        d_h0 = None
        if ctx.h0_shape is not None:
            d_h0 = torch.zeros((ctx.shape[0],) + ctx.h0_shape[1:], dtype=torch.float32, device=ctx.device)
        for (lo, hi), st in zip(ctx.spans, ctx.states):
            g_o = d_o[lo:hi] if d_o is not None else torch.zeros((hi - lo,) + ctx.shape[1:], dtype=ctx.dtype,
                                                                 device=ctx.device)
            op.prepare_bwd(st, g_o, [g[lo:hi] for g in grads])
        # same group order as the forward, so that neighbouring ranks overlap in the reverse chain too
        for (lo, hi), st in zip(ctx.spans, ctx.states):
            # the gradient of this rank's boundary state: what the right neighbour sends, plus whatever the
            # caller's loss puts on the local final state
            d_state = None if d_ht is None else d_ht[lo:hi].to(torch.float32)
            if ctx.next_rank is not None:
                recv = torch.empty((hi - lo,) + ctx.state_tail, dtype=torch.float32, device=ctx.device)
                dist.recv(recv, src=ctx.next_rank, group=ctx.group)
                d_state = recv if d_state is None else recv + d_state
            d_hin = op.scan_bwd(st, d_state)
            if ctx.prev_rank is not None:
                dist.send(d_hin.contiguous(), dst=ctx.prev_rank, group=ctx.group)
            elif d_h0 is not None:
                d_h0[lo:hi] = d_hin
        for (lo, hi), st in zip(ctx.spans, ctx.states):
            res = op.finish_bwd(st)
            for i in range(6):
                if res[i].data_ptr() != grads[i][lo:hi].data_ptr():
                    grads[i][lo:hi] = res[i]
        if d_h0 is not None and ctx.h0_shape[0] == 1:
            d_h0 = d_h0.sum(0, keepdim=True)
        ctx.states = None
        return (*grads, d_h0, None, None, None, None)


def generalized_delta_rule_sp(r, w, k, v, a, b, initial_state: Optional[torch.Tensor] = None,
                              output_final_state: bool = True, head_first: bool = False,
                              group=None, pipeline_groups: Optional[int] = None, local_op=None):
    """``generalized_delta_rule`` on a sequence split across the ranks of ``group`` (rank order =
    sequence order).  Every rank passes its own slice of the token tensors; ``initial_state`` is used on
    the first rank only.  Returns the local slice of ``o`` and, when ``output_final_state``, the state at
    the end of the local slice (the true final state on the last rank; a loss on the state of another rank
    is differentiated too).

    ``pipeline_groups``: the batch rows are cut into this many groups whose scans follow one another, so that
    a rank scans group j + 1 while its right neighbour scans group j (the chain then costs about
    ``(ranks + groups - 1) / (ranks * groups)`` of the unsplit scans).  Default: up to 4 groups of at least 256
    (batch, head) units each, enough to fill the scan kernels' grid.

    ``local_op``: a ``PhasedLocalOp``, or a ``generalized_delta_rule``-like callable (run as a plain chain);
    default: the phased tensor-core operator for bfloat16 CUDA tensors, else the plain chain over
    ``rwkv_ops_b200.generalized_delta_rule``.
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    B = r.shape[0]
    if pipeline_groups is None:
        H = r.shape[1] if head_first else r.shape[2]
        pipeline_groups = min(4, (B * H) // 256)
    groups = max(1, min(int(pipeline_groups), B))
    if local_op is None:
        op = ChunkedPhasedOp() if (r.is_cuda and r.dtype == torch.bfloat16) else ChainPhasedOp(_default_local_op())
    elif isinstance(local_op, PhasedLocalOp):
        op = local_op
    else:
        op = ChainPhasedOp(local_op)
    o, ht = _Chain.apply(r, w, k, v, a, b, initial_state, bool(head_first), group, op, groups)
    return (o, ht) if output_final_state else o
