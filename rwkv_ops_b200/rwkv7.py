"""RWKV7 generalized delta rule: the reference's Python interface over the CUDA library.

Mirrors ``generalized_delta_rule`` and ``get_generalized_delta_rule`` of the reference
(``rwkv_ops/rwkv7_kernel/native_keras_op.py:23-95``, ``rwkv_ops/rwkv7_kernel/torch_op.py:458-490``,
``rwkv_ops/rwkv7_kernel/__init__.py:14-156``): same argument names and meaning, ``exp(-exp(w))``
decay, output in ``r``'s dtype, float32 states in the native ``[N, H, V, K]`` layout, a bare
tensor when ``output_final_state`` is false.  The work is done by ``torch.library`` custom ops
with autograd that call the C ABI through ctypes; there is no Triton, no multi-backend dispatch
and no CPU fallback.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _lib

HEAD_SIZE = 64               # the head size of the tensor-core path
HEAD_SIZES = (64, 128)       # head sizes the operator accepts (128: float32 recurrence for every dtype)
_ALGO_NAMES = {"auto": _lib.ALGO_AUTO, "recurrent": _lib.ALGO_RECURRENT, "chunked": _lib.ALGO_CHUNKED}


def _default_algo() -> int:
    return _ALGO_NAMES[os.environ.get("RWKV_OPS_B200_RWKV7_ALGO", "auto").lower()]


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def _keep_limit_bytes(device) -> int:
    """Largest per-call tile store that a training forward may hand to its backward instead of having
    the backward recompute the forward: ``RWKV_OPS_B200_KEEP_LIMIT_MB`` (MiB) when set, else a quarter
    of the device's memory (about 45 GiB on a B200)."""
    env = os.environ.get("RWKV_OPS_B200_KEEP_LIMIT_MB")
    if env is not None:
        return int(env) << 20
    return torch.cuda.get_device_properties(device).total_memory // 4


# --------------------------------------------------------------------------------------------
# custom ops (tensors are contiguous token tensors of one dtype; states float32)
# --------------------------------------------------------------------------------------------
@torch.library.custom_op("rwkv_ops_b200::rwkv7_fwd", mutates_args=())
def _rwkv7_fwd(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
               b: torch.Tensor, h0: Optional[torch.Tensor], head_first: bool, algo: int
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, h0)
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    code = _lib.dtype_code(r.dtype)
    o = torch.empty_like(r)
    ht = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        if T == 1:
            rc = lib.rwkvb200_rwkv7_step(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                         b.data_ptr(), _lib.ptr(h0), n_state, ht.data_ptr(), o.data_ptr(),
                                         B, H, K, code, _lib.stream_ptr(dev))
            _lib.check(rc, "rwkv7_step")
            _lib.check_status("rwkv7_step")
        else:
            nws = lib.rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, K, code, algo)
            ws = _workspace(nws, dev)
            rc = lib.rwkvb200_rwkv7_fwd(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                        b.data_ptr(), _lib.ptr(h0), n_state, o.data_ptr(), ht.data_ptr(),
                                        _lib.ptr(ws), nws, B, T, H, K, code, int(head_first), algo,
                                        _lib.stream_ptr(dev))
            _lib.check(rc, "rwkv7_fwd")
            _lib.check_status("rwkv7_fwd")
    return o, ht


@_rwkv7_fwd.register_fake
def _(r, w, k, v, a, b, h0, head_first, algo):
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    return torch.empty_like(r), r.new_empty((B, H, K, K), dtype=torch.float32)


# Training forward of the chunked path: same results, and the per-chunk tiles the backward needs are
# returned in `kept` (an opaque byte tensor) so that the backward does not recompute the forward.
@torch.library.custom_op("rwkv_ops_b200::rwkv7_fwd_keep", mutates_args=())
def _rwkv7_fwd_keep(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                    b: torch.Tensor, h0: Optional[torch.Tensor], head_first: bool, algo: int
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, h0)
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    code = _lib.dtype_code(r.dtype)
    o = torch.empty_like(r)
    ht = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    flags = algo | _lib.ALGO_KEEP
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, K, code, flags)
        kept = torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_rwkv7_fwd(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                    b.data_ptr(), _lib.ptr(h0), n_state, o.data_ptr(), ht.data_ptr(),
                                    kept.data_ptr(), nws, B, T, H, K, code, int(head_first), flags,
                                    _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_fwd")
        _lib.check_status("rwkv7_fwd")
    return o, ht, kept


@_rwkv7_fwd_keep.register_fake
def _(r, w, k, v, a, b, h0, head_first, algo):
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    return (torch.empty_like(r), r.new_empty((B, H, K, K), dtype=torch.float32),
            r.new_empty((_lib.rwkv7_kept_bytes(B, T, H),), dtype=torch.uint8))


# `kept` also serves as scratch for the backward kernels; the tiles the forward left in it are not changed.
# (Not declared in mutates_args: autograd would then refuse a second backward through the same graph, and
# nothing that anyone reads from `kept` ever changes.)
@torch.library.custom_op("rwkv_ops_b200::rwkv7_bwd_kept", mutates_args=())
def _rwkv7_bwd_kept(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                    b: torch.Tensor, h0: Optional[torch.Tensor], d_o: torch.Tensor, d_ht: Optional[torch.Tensor],
                    kept: torch.Tensor, head_first: bool, algo: int
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                               torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, h0, d_o, d_ht, kept)
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    code = _lib.dtype_code(r.dtype)
    dr, dw, dk, dv, da, db = (torch.empty_like(r) for _ in range(6))
    dh0 = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        rc = lib.rwkvb200_rwkv7_bwd(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                    b.data_ptr(), _lib.ptr(h0), n_state, d_o.data_ptr(), _lib.ptr(d_ht),
                                    dr.data_ptr(), dw.data_ptr(), dk.data_ptr(), dv.data_ptr(), da.data_ptr(),
                                    db.data_ptr(), dh0.data_ptr(), kept.data_ptr(), kept.numel(),
                                    B, T, H, K, code, int(head_first), algo | _lib.ALGO_KEEP, _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_bwd")
        _lib.check_status("rwkv7_bwd")
    return dr, dw, dk, dv, da, db, dh0


@_rwkv7_bwd_kept.register_fake
def _(r, w, k, v, a, b, h0, d_o, d_ht, kept, head_first, algo):
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    e = torch.empty_like
    return e(r), e(r), e(r), e(r), e(r), e(r), r.new_empty((B, H, K, K), dtype=torch.float32)


def _setup_ctx_keep(ctx, inputs, output):
    r, w, k, v, a, b, h0, head_first, algo = inputs
    ctx.save_for_backward(r, w, k, v, a, b, h0, output[2])
    ctx.set_materialize_grads(False)   # no zero tensor for the (never differentiated) tile store
    ctx.head_first = head_first
    ctx.algo = algo


def _backward_keep(ctx, d_o, d_ht, d_kept):
    r, w, k, v, a, b, h0, kept = ctx.saved_tensors
    if d_o is None:
        d_o = torch.zeros_like(r)
    d_o = d_o.to(r.dtype).contiguous()
    if d_ht is not None:
        d_ht = d_ht.to(torch.float32).contiguous()
    dr, dw, dk, dv, da, db, dh0 = _rwkv7_bwd_kept(r, w, k, v, a, b, h0, d_o, d_ht, kept, ctx.head_first, ctx.algo)
    if h0 is None or not ctx.needs_input_grad[6]:
        dh0 = None
    elif h0.shape[0] == 1 and dh0.shape[0] != 1:
        dh0 = dh0.sum(0, keepdim=True)
    return dr, dw, dk, dv, da, db, dh0, None, None


torch.library.register_autograd("rwkv_ops_b200::rwkv7_fwd_keep", _backward_keep, setup_context=_setup_ctx_keep)


@torch.library.custom_op("rwkv_ops_b200::rwkv7_bwd", mutates_args=())
def _rwkv7_bwd(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
               b: torch.Tensor, h0: Optional[torch.Tensor], d_o: torch.Tensor, d_ht: Optional[torch.Tensor],
               head_first: bool, algo: int
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                          torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, h0, d_o, d_ht)
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    code = _lib.dtype_code(r.dtype)
    dr, dw, dk, dv, da, db = (torch.empty_like(r) for _ in range(6))
    dh0 = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_bwd_workspace_bytes(B, T, H, K, code, algo)
        ws = _workspace(nws, dev)
        rc = lib.rwkvb200_rwkv7_bwd(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                    b.data_ptr(), _lib.ptr(h0), n_state, d_o.data_ptr(), _lib.ptr(d_ht),
                                    dr.data_ptr(), dw.data_ptr(), dk.data_ptr(), dv.data_ptr(), da.data_ptr(),
                                    db.data_ptr(), dh0.data_ptr(), _lib.ptr(ws), nws,
                                    B, T, H, K, code, int(head_first), algo, _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_bwd")
        _lib.check_status("rwkv7_bwd")
    return dr, dw, dk, dv, da, db, dh0


@_rwkv7_bwd.register_fake
def _(r, w, k, v, a, b, h0, d_o, d_ht, head_first, algo):
    if head_first:
        B, H, T, K = r.shape
    else:
        B, T, H, K = r.shape
    e = torch.empty_like
    return e(r), e(r), e(r), e(r), e(r), e(r), r.new_empty((B, H, K, K), dtype=torch.float32)


def _setup_ctx(ctx, inputs, output):
    r, w, k, v, a, b, h0, head_first, algo = inputs
    ctx.save_for_backward(r, w, k, v, a, b, h0)
    ctx.set_materialize_grads(False)
    ctx.head_first = head_first
    ctx.algo = algo


def _backward(ctx, d_o, d_ht):
    r, w, k, v, a, b, h0 = ctx.saved_tensors
    if d_o is None:
        d_o = torch.zeros_like(r)
    d_o = d_o.to(r.dtype).contiguous()
    if d_ht is not None:
        d_ht = d_ht.to(torch.float32).contiguous()
    dr, dw, dk, dv, da, db, dh0 = _rwkv7_bwd(r, w, k, v, a, b, h0, d_o, d_ht, ctx.head_first, ctx.algo)
    if h0 is None or not ctx.needs_input_grad[6]:
        dh0 = None
    elif h0.shape[0] == 1 and dh0.shape[0] != 1:
        dh0 = dh0.sum(0, keepdim=True)   # one state broadcast over the batch
    return dr, dw, dk, dv, da, db, dh0, None, None


torch.library.register_autograd("rwkv_ops_b200::rwkv7_fwd", _backward, setup_context=_setup_ctx)


# --------------------------------------------------------------------------------------------
# public interface
# --------------------------------------------------------------------------------------------
def generalized_delta_rule(
    r: torch.Tensor,
    w: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = True,
    head_first: bool = False,
):
    """Drop-in for the reference's ``generalized_delta_rule``.

    ``r, w, k, v, a, b``: ``[B, T, H, K]`` (``[B, H, T, K]`` when ``head_first``) with head size
    ``K`` 64 or 128 (the reference's value test runs 128, ``test_script/test_rwkv7_value.py:46-51``), any
    of float32 / bfloat16 / float16; ``w`` is the raw decay input (the operator applies
    ``exp(-exp(w))``).  ``initial_state``: float32 ``[N, H, K, K]`` with ``N == B`` or ``N == 1``
    (broadcast), value index before key index.  Returns ``(o, final_state)`` or just ``o``.
    Head size 64 with bfloat16 tokens takes the tensor-core path, everything else the float32 recurrence
    (``RWKV_OPS_B200_RWKV7_ALGO=chunked`` sends float32 / float16 tokens of head size 64 through the tensor-core
    path as well, rounded to bfloat16).
    """
    _lib.require_cuda(r, w, k, v, a, b, initial_state)
    if r.dim() != 4 or r.shape[-1] not in HEAD_SIZES:
        raise ValueError(f"expected 4-D token tensors with head size in {HEAD_SIZES}, got {tuple(r.shape)}")
    HEAD_SIZE = r.shape[-1]
    for name, x in (("w", w), ("k", k), ("v", v), ("a", a), ("b", b)):
        if x.shape != r.shape:
            raise ValueError(f"{name} has shape {tuple(x.shape)}, expected {tuple(r.shape)}")
    out_dtype = r.dtype
    cdt = r.dtype if r.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    if cdt != torch.bfloat16 and HEAD_SIZE == 64 and _default_algo() == _lib.ALGO_CHUNKED:
        # RWKV_OPS_B200_RWKV7_ALGO=chunked asked for the tensor-core path by name: float32 / float16 tokens are
        # rounded to bfloat16 for it (about 15 times the speed of the float32 recurrence at bfloat16-operand
        # accuracy, 2e-2 against the oracle instead of 1e-4); gradients come back in the inputs' dtypes
        cdt = torch.bfloat16
    r_, w_, k_, v_, a_, b_ = (x.to(cdt).contiguous() for x in (r, w, k, v, a, b))
    B = r.shape[0]
    H = r.shape[1] if head_first else r.shape[2]
    h0 = None
    if initial_state is not None:
        if initial_state.dim() != 4 or tuple(initial_state.shape[1:]) != (H, HEAD_SIZE, HEAD_SIZE) \
                or initial_state.shape[0] not in (1, B):
            raise ValueError(
                f"initial_state must be [B or 1, {H}, {HEAD_SIZE}, {HEAD_SIZE}], got {tuple(initial_state.shape)}")
        h0 = initial_state.to(torch.float32).contiguous()
    algo = _default_algo()
    T = r.shape[2] if head_first else r.shape[1]
    needs_grad = torch.is_grad_enabled() and (
        any(x.requires_grad for x in (r_, w_, k_, v_, a_, b_)) or (h0 is not None and h0.requires_grad))
    keep = False
    if needs_grad and T > 1 and cdt == torch.bfloat16 and HEAD_SIZE == 64 and algo in (_lib.ALGO_AUTO, _lib.ALGO_CHUNKED):
        nws = _lib.load().rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, HEAD_SIZE, _lib.BF16, algo | _lib.ALGO_KEEP)
        keep = nws <= _keep_limit_bytes(r_.device)
    if keep:
        o, ht, _ = _rwkv7_fwd_keep(r_, w_, k_, v_, a_, b_, h0, bool(head_first), algo)
    else:
        o, ht = _rwkv7_fwd(r_, w_, k_, v_, a_, b_, h0, bool(head_first), algo)
    if o.dtype != out_dtype:
        o = o.to(out_dtype)
    if output_final_state:
        return o, ht
    return o


def get_generalized_delta_rule(HEAD_SIZE: int = 64, KERNEL_TYPE: str = "cuda"):
    """Reference signature (``rwkv_ops/rwkv7_kernel/__init__.py:14``): returns ``(fn, USE_KERNEL)``.

    ``USE_KERNEL`` is always True (callers use it to choose the padding recipe of the kernel
    path).  ``KERNEL_TYPE`` is accepted for compatibility and ignored: there is one implementation.
    """
    if HEAD_SIZE not in HEAD_SIZES:
        raise ValueError(f"rwkv_ops_b200 is built for head sizes {HEAD_SIZES}")
    return generalized_delta_rule, True
