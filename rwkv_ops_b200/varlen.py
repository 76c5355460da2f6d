"""RWKV7 generalized delta rule on packed variable-length batches.

The reference carries ``cu_seqlens`` plumbing for this in its Triton path but has it disabled
(``rwkv_ops/rwkv7_kernel/torch_op.py:283,299``, the ``if False:`` blocks of e.g.
``triton_kernel/chunk_A_fwd.py:47-56``); its users pad every sequence to the longest one and push the
padding's decay input to ``-1e9`` (``README.md:92-98``).  ``generalized_delta_rule_varlen`` takes the
sequences laid end to end instead -- token tensors ``[1, total_len, H, 64]`` plus ``cu_seqlens``
``[n_seq + 1]`` (``cu_seqlens[i]`` is the first token of sequence ``i``) -- and returns what running the
operator on every sequence alone would: ``o`` ``[1, total_len, H, 64]`` and one final state per
sequence ``[n_seq, H, 64, 64]``.  No padded token is ever loaded or stored.

bfloat16 token tensors run on the chunked tensor-core kernels (chunk slots past the end of a sequence
are skipped, a partial last chunk is stored row by row so that the next sequence's rows stay intact);
other dtypes run the dense operator once per sequence.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .rwkv7 import HEAD_SIZE, generalized_delta_rule


def _seq_arrays(cu_seqlens, total_len: int, device):
    cu = torch.as_tensor(cu_seqlens).detach().to("cpu", torch.int64).flatten()
    if cu.numel() < 2 or int(cu[0]) != 0 or int(cu[-1]) != total_len:
        raise ValueError(f"cu_seqlens must run from 0 to the number of tokens ({total_len}), got {cu.tolist()}")
    lens = cu[1:] - cu[:-1]
    if int(lens.min()) < 1:
        raise ValueError("every sequence must hold at least one token")
    start = cu[:-1].to(device=device, dtype=torch.int32)
    return cu, start, lens.to(device=device, dtype=torch.int32), int(lens.max())


class PackedSequences:
    """``cu_seqlens`` prepared once (host copy, device arrays of first tokens and lengths, longest length)
    for all the calls that share it, e.g. every layer of a step; pass it in place of ``cu_seqlens``."""

    def __init__(self, cu_seqlens, device="cuda"):
        cu = torch.as_tensor(cu_seqlens).detach().to("cpu", torch.int64).flatten()
        self.total_len = int(cu[-1]) if cu.numel() else 0
        self.device = torch.device(device)
        self.cu, self.start, self.lens, self.max_len = _seq_arrays(cu, self.total_len, self.device)


@torch.library.custom_op("rwkv_ops_b200::rwkv7_fwd_varlen", mutates_args=())
def _fwd_varlen(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                b: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_len: int,
                h0: Optional[torch.Tensor], keep: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, seq_start, seq_len, h0)
    _, T, H, K = r.shape
    n_seq = seq_start.numel()
    o = torch.empty_like(r)
    ht = torch.empty(n_seq, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_varlen_workspace_bytes(n_seq, max_len, H, K, int(keep))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_rwkv7_fwd_varlen(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                           b.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(), n_seq, max_len,
                                           T, _lib.ptr(h0), n_state, o.data_ptr(), ht.data_ptr(), ws.data_ptr(),
                                           nws, H, K, _lib.dtype_code(r.dtype), int(keep), _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_fwd_varlen")
        _lib.check_status("rwkv7_fwd_varlen")
    return o, ht, (ws if keep else ws.new_empty((1,)))


@_fwd_varlen.register_fake
def _(r, w, k, v, a, b, seq_start, seq_len, max_len, h0, keep):
    _, T, H, K = r.shape
    n_seq = seq_start.numel()
    return (torch.empty_like(r), r.new_empty((n_seq, H, K, K), dtype=torch.float32),
            r.new_empty((_lib.rwkv7_kept_bytes(n_seq, max_len, H) if keep else 1,), dtype=torch.uint8))


# `kept` also serves as scratch for the backward kernels; the tiles the forward left in it are not changed.
@torch.library.custom_op("rwkv_ops_b200::rwkv7_bwd_varlen", mutates_args=())
def _bwd_varlen(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                b: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_len: int,
                h0: Optional[torch.Tensor], d_o: torch.Tensor, d_ht: Optional[torch.Tensor], kept: torch.Tensor
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                           torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, seq_start, seq_len, h0, d_o, d_ht, kept)
    _, T, H, K = r.shape
    n_seq = seq_start.numel()
    dr, dw, dk, dv, da, db = (torch.empty_like(r) for _ in range(6))
    dh0 = torch.empty(n_seq, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_varlen_workspace_bytes(n_seq, max_len, H, K, 1)
        have = kept.numel() >= nws
        ws = kept if have else torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_rwkv7_bwd_varlen(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                           b.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(), n_seq, max_len,
                                           T, _lib.ptr(h0), n_state, d_o.data_ptr(), _lib.ptr(d_ht),
                                           dr.data_ptr(), dw.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                           da.data_ptr(), db.data_ptr(), dh0.data_ptr(), ws.data_ptr(), nws,
                                           H, K, _lib.dtype_code(r.dtype), int(have), _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_bwd_varlen")
        _lib.check_status("rwkv7_bwd_varlen")
    return dr, dw, dk, dv, da, db, dh0


@_bwd_varlen.register_fake
def _(r, w, k, v, a, b, seq_start, seq_len, max_len, h0, d_o, d_ht, kept):
    _, T, H, K = r.shape
    e = torch.empty_like
    return e(r), e(r), e(r), e(r), e(r), e(r), r.new_empty((seq_start.numel(), H, K, K), dtype=torch.float32)


def _setup_ctx(ctx, inputs, output):
    r, w, k, v, a, b, seq_start, seq_len, max_len, h0, keep = inputs
    ctx.save_for_backward(r, w, k, v, a, b, seq_start, seq_len, h0, output[2])
    ctx.set_materialize_grads(False)
    ctx.max_len = max_len


def _backward(ctx, d_o, d_ht, d_kept):
    r, w, k, v, a, b, seq_start, seq_len, h0, kept = ctx.saved_tensors
    if d_o is None:
        d_o = torch.zeros_like(r)
    d_o = d_o.to(r.dtype).contiguous()
    if d_ht is not None:
        d_ht = d_ht.to(torch.float32).contiguous()
    dr, dw, dk, dv, da, db, dh0 = _bwd_varlen(r, w, k, v, a, b, seq_start, seq_len, ctx.max_len, h0, d_o, d_ht, kept)
    if h0 is None or not ctx.needs_input_grad[9]:
        dh0 = None
    elif h0.shape[0] == 1 and dh0.shape[0] != 1:
        dh0 = dh0.sum(0, keepdim=True)   # one state broadcast over the sequences
    return dr, dw, dk, dv, da, db, None, None, None, dh0, None


torch.library.register_autograd("rwkv_ops_b200::rwkv7_fwd_varlen", _backward, setup_context=_setup_ctx)


def _token_args(r, w, k, v, a, b):
    """The six token tensors in ``r``'s dtype, contiguous: the kernels read all of them as one element type
    (``generalized_delta_rule`` casts in the same way; under mixed precision ``w`` often arrives as float32)."""
    return [x.to(r.dtype).contiguous() for x in (r, w, k, v, a, b)]


def generalized_delta_rule_varlen(r, w, k, v, a, b, cu_seqlens, initial_state=None, output_final_state=True):
    """``generalized_delta_rule`` over sequences packed end to end (see the module docstring).

    ``r, w, k, v, a, b``: ``[1, total_len, H, 64]``; ``cu_seqlens``: ``n_seq + 1`` increasing integers from
    0 to ``total_len`` (tensor or list, or a ``PackedSequences`` made from them once); ``initial_state``: float32 ``[n_seq or 1, H, 64, 64]``.
    Returns ``(o, final_state)`` with ``final_state`` ``[n_seq, H, 64, 64]``, or just ``o``.
    """
    dev = _lib.require_cuda(r, w, k, v, a, b, initial_state)
    if r.dim() != 4 or r.shape[0] != 1 or r.shape[-1] != HEAD_SIZE:
        raise ValueError(f"expected packed token tensors [1, total_len, H, {HEAD_SIZE}], got {tuple(r.shape)}")
    for name, x in (("w", w), ("k", k), ("v", v), ("a", a), ("b", b)):
        if x.shape != r.shape:
            raise ValueError(f"{name} has shape {tuple(x.shape)}, expected {tuple(r.shape)}")
    T, H = r.shape[1], r.shape[2]
    if isinstance(cu_seqlens, PackedSequences):
        if cu_seqlens.total_len != T or cu_seqlens.start.device != dev:
            raise ValueError("the PackedSequences object was made for another token count or device")
        cu, start, lens, max_len = cu_seqlens.cu, cu_seqlens.start, cu_seqlens.lens, cu_seqlens.max_len
    else:
        cu, start, lens, max_len = _seq_arrays(cu_seqlens, T, dev)
    n_seq = start.numel()
    h0 = None
    if initial_state is not None:
        if initial_state.dim() != 4 or tuple(initial_state.shape[1:]) != (H, HEAD_SIZE, HEAD_SIZE) \
                or initial_state.shape[0] not in (1, n_seq):
            raise ValueError(f"initial_state must be [{n_seq} or 1, {H}, {HEAD_SIZE}, {HEAD_SIZE}], "
                             f"got {tuple(initial_state.shape)}")
        h0 = initial_state.to(torch.float32).contiguous()

    if r.dtype != torch.bfloat16:
        # one dense call per sequence (the float32 recurrence has no packed form)
        outs, states = [], []
        for i in range(n_seq):
            s, e = int(cu[i]), int(cu[i + 1])
            hi = None if h0 is None else h0[i:i + 1] if h0.shape[0] == n_seq else h0
            oi, si = generalized_delta_rule(*(x[:, s:e] for x in (r, w, k, v, a, b)), initial_state=hi)
            outs.append(oi)
            states.append(si)
        o, ht = torch.cat(outs, dim=1), torch.cat(states, dim=0)
    else:
        args = _token_args(r, w, k, v, a, b)
        needs_grad = torch.is_grad_enabled() and (
            any(x.requires_grad for x in args) or (h0 is not None and h0.requires_grad))
        o, ht, _ = _fwd_varlen(*args, start, lens, max_len, h0, needs_grad)
    return (o, ht) if output_final_state else o


# ---------------------------------------------------------------------------------------------------------
# RWKV6 wkv on packed batches
# ---------------------------------------------------------------------------------------------------------
@torch.library.custom_op("rwkv_ops_b200::wkv6_fwd_varlen", mutates_args=())
def _wkv6_fwd_varlen(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
                     seq_start: torch.Tensor, seq_len: torch.Tensor, max_len: int, s0: Optional[torch.Tensor],
                     state_map: Optional[torch.Tensor], keep: bool
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, k, v, w, u, seq_start, seq_len, s0, state_map)
    T = r.shape[1]
    H, N = u.shape
    n_seq = seq_start.numel()
    code = _lib.dtype_code(r.dtype)
    y = torch.empty_like(r)
    sT = torch.empty(n_seq, H, N, N, dtype=torch.float32, device=dev)
    n_state = 0 if s0 is None else s0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_wkv6_varlen_workspace_bytes(n_seq, max_len, H, N, code, int(keep))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_wkv6_fwd_varlen(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                          seq_start.data_ptr(), seq_len.data_ptr(), n_seq, max_len, T,
                                          _lib.ptr(s0), n_state, _lib.ptr(state_map), y.data_ptr(), sT.data_ptr(),
                                          ws.data_ptr(), nws, H, N, code, int(keep), _lib.stream_ptr(dev))
        _lib.check(rc, "wkv6_fwd_varlen")
        _lib.check_status("wkv6_fwd_varlen")
    return y, sT, (ws if keep else ws.new_empty((1,)))


@_wkv6_fwd_varlen.register_fake
def _(r, k, v, w, u, seq_start, seq_len, max_len, s0, state_map, keep):
    H, N = u.shape
    n_seq = seq_start.numel()
    return (torch.empty_like(r), r.new_empty((n_seq, H, N, N), dtype=torch.float32),
            r.new_empty((_lib.wkv6_kept_bytes(n_seq, max_len, H) if keep else 1,), dtype=torch.uint8))


# `kept` also serves as scratch for the backward kernel; the states the forward left in it are not changed.
@torch.library.custom_op("rwkv_ops_b200::wkv6_bwd_varlen", mutates_args=())
def _wkv6_bwd_varlen(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
                     seq_start: torch.Tensor, seq_len: torch.Tensor, max_len: int, s0: Optional[torch.Tensor],
                     state_map: Optional[torch.Tensor], d_y: torch.Tensor, d_sT: Optional[torch.Tensor],
                     kept: torch.Tensor
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, k, v, w, u, seq_start, seq_len, s0, state_map, d_y, d_sT, kept)
    T = r.shape[1]
    H, N = u.shape
    n_seq = seq_start.numel()
    code = _lib.dtype_code(r.dtype)
    dr, dk, dv, dw = (torch.empty_like(r) for _ in range(4))
    du = torch.empty(H, N, dtype=torch.float32, device=dev)
    ds0 = torch.empty(n_seq, H, N, N, dtype=torch.float32, device=dev)
    n_state = 0 if s0 is None else s0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_wkv6_varlen_workspace_bytes(n_seq, max_len, H, N, code, 1)
        have = kept.numel() >= nws
        ws = kept if have else torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_wkv6_bwd_varlen(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                          seq_start.data_ptr(), seq_len.data_ptr(), n_seq, max_len, T,
                                          _lib.ptr(s0), n_state, _lib.ptr(state_map), d_y.data_ptr(),
                                          _lib.ptr(d_sT), dr.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                          dw.data_ptr(), du.data_ptr(), ds0.data_ptr(), ws.data_ptr(), nws,
                                          H, N, code, int(have), _lib.stream_ptr(dev))
        _lib.check(rc, "wkv6_bwd_varlen")
        _lib.check_status("wkv6_bwd_varlen")
    return dr, dk, dv, dw, du, ds0


@_wkv6_bwd_varlen.register_fake
def _(r, k, v, w, u, seq_start, seq_len, max_len, s0, state_map, d_y, d_sT, kept):
    H, N = u.shape
    e = torch.empty_like
    return (e(r), e(r), e(r), e(r), r.new_empty((H, N), dtype=torch.float32),
            r.new_empty((seq_start.numel(), H, N, N), dtype=torch.float32))


def _wkv6_setup_ctx(ctx, inputs, output):
    r, k, v, w, u, seq_start, seq_len, max_len, s0, state_map, keep = inputs
    ctx.save_for_backward(r, k, v, w, u, seq_start, seq_len, s0, state_map, output[2])
    ctx.set_materialize_grads(False)
    ctx.max_len = max_len


def _wkv6_backward(ctx, d_y, d_sT, d_kept):
    r, k, v, w, u, seq_start, seq_len, s0, state_map, kept = ctx.saved_tensors
    if d_y is None:
        d_y = torch.zeros_like(r)
    d_y = d_y.to(r.dtype).contiguous()
    if d_sT is not None:
        d_sT = d_sT.to(torch.float32).contiguous()
    dr, dk, dv, dw, du, ds0_rows = _wkv6_bwd_varlen(r, k, v, w, u, seq_start, seq_len, ctx.max_len, s0, state_map,
                                                    d_y, d_sT, kept)
    ds0 = None
    if s0 is not None and ctx.needs_input_grad[8]:
        n_state, n_seq = s0.shape[0], seq_start.numel()
        if state_map is not None:
            idx = state_map.to(torch.int64)
        elif n_state == 1:
            idx = torch.zeros(n_seq, dtype=torch.int64, device=r.device)
        else:
            idx = torch.arange(n_seq, device=r.device)
        ds0 = torch.zeros_like(s0).index_add_(0, idx, ds0_rows)      # sequences that share a table row add up
    return dr, dk, dv, dw, du, None, None, None, ds0, None, None


torch.library.register_autograd("rwkv_ops_b200::wkv6_fwd_varlen", _wkv6_backward, setup_context=_wkv6_setup_ctx)


def wkv6_varlen(r, k, v, w, u, cu_seqlens, init_state=None, state_map=None, head_size: int = 64):
    """The RWKV6 wkv operator over sequences packed end to end.

    The reference's operator takes dense ``[B, T, C]`` batches only (``rwkv_ops/rwkv6_kernel/
    ops_rwkv_kernel.py:10-21``); this is the same recurrence per sequence without a padded token ever loaded,
    computed or stored.  ``r, k, v, w``: ``[1, total_len, C]`` (or ``[total_len, C]``), ``C = H * 64``;
    ``u``: ``C`` elements; ``cu_seqlens``: ``n_seq + 1`` increasing integers from 0 to ``total_len`` (tensor,
    list or ``PackedSequences``); ``init_state``: ``[n_state, H, 64, 64]`` or ``[H, 64, 64]`` and ``state_map``
    ``[n_seq]`` as in the dense operator, with the sequence in the place of the batch row.  Returns
    ``(y, state)``: ``y`` shaped like ``r``, ``state`` ``[n_seq, H, 64, 64]`` in the operator's state dtype.
    Differentiable with respect to ``r, k, v, w, u`` and ``init_state``.
    """
    dev = _lib.require_cuda(r, k, v, w, u, init_state)
    if head_size != 64:
        raise ValueError("the packed wkv6 operator is built for head size 64")
    squeeze = r.dim() == 2
    if squeeze:
        r, k, v, w = (x[None] for x in (r, k, v, w))
    if r.dim() != 3 or r.shape[0] != 1 or r.shape[-1] % 64:
        raise ValueError(f"expected packed token tensors [1, total_len, H*64], got {tuple(r.shape)}")
    for name, x in (("k", k), ("v", v), ("w", w)):
        if x.shape != r.shape or x.dtype != r.dtype:
            raise ValueError(f"{name} must match r in shape and dtype")
    T, C = r.shape[1], r.shape[2]
    H, N = C // 64, 64
    if u.numel() != C:
        raise ValueError(f"u must have {C} elements")
    if isinstance(cu_seqlens, PackedSequences):
        if cu_seqlens.total_len != T or cu_seqlens.start.device != dev:
            raise ValueError("the PackedSequences object was made for another token count or device")
        start, lens, max_len = cu_seqlens.start, cu_seqlens.lens, cu_seqlens.max_len
    else:
        _, start, lens, max_len = _seq_arrays(cu_seqlens, T, dev)
    n_seq = start.numel()
    dt = r.dtype
    cdt = dt if dt in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    state_dtype = torch.float32 if dt == torch.float16 else dt
    s0 = smap = None
    if init_state is not None:
        if init_state.dim() == 3:
            init_state = init_state[None]
        if init_state.dim() != 4 or tuple(init_state.shape[1:]) != (H, N, N):
            raise ValueError(f"init_state must be [n_state, {H}, {N}, {N}] or [{H}, {N}, {N}]")
        n_state = init_state.shape[0]
        if state_map is None:
            if n_state not in (1, n_seq):
                raise ValueError("state_map cannot be inferred from init_state; pass it explicitly")
        else:
            if isinstance(state_map, (list, tuple)):
                state_map = torch.tensor(state_map, dtype=torch.int32)
            if state_map.numel() != n_seq:
                raise ValueError("state_map must have one entry per sequence")
            if not state_map.is_cuda and not (bool((state_map >= 0).all()) and bool((state_map < n_state).all())):
                raise ValueError(f"state_map values must lie in [0, {n_state})")
            smap = state_map.to(device=dev, dtype=torch.int32).contiguous().view(n_seq)
        s0 = init_state.to(torch.float32).contiguous()
    elif state_map is not None:
        raise ValueError("state_map needs init_state")
    args = [x.to(cdt).contiguous() for x in (r, k, v, w)]
    uu = u.reshape(H, N).to(torch.float32).contiguous()
    needs_grad = torch.is_grad_enabled() and (
        any(x.requires_grad for x in (r, k, v, w, u)) or (init_state is not None and init_state.requires_grad))
    y, sT, _ = _wkv6_fwd_varlen(*args, uu, start, lens, max_len, s0, smap, needs_grad)
    if y.dtype != dt:
        y = y.to(dt)
    if squeeze:
        y = y[0]
    return y, sT.to(state_dtype)
