"""RWKV7 delta rule with the elementwise producers of its ``w``, ``a`` and ``b`` inputs fused in.

In an RWKV7 time-mix block three of the operator's six inputs are elementwise functions of
pre-activations that exist only to feed it -- with the input distributions of the reference's value test
(``test_script/test_rwkv7_value.py``): ``w = -exp(-1/2) * sigmoid(w_pre)``, ``kk = normalize(kk_pre)``
over the 64 channels of a head, ``a = -kk``, ``b = kk * sigmoid(a_pre)``.  Computed by separate kernels
they cost a write and a read of three ``[B, T, H, 64]`` tensors in the forward pass and as much again for
their gradients in the backward pass.  ``generalized_delta_rule_fused`` takes the pre-activations and
computes the three inputs where the operator's first kernel loads them; its backward pass returns the
gradients of the pre-activations.  ``w``, ``a`` and ``b`` are rounded to bfloat16 exactly as materialised
tensors would be, so the result equals ``generalized_delta_rule(r, w, k, v, a, b)`` bit for bit.

bfloat16 tensors ``[B, T, H, 64]`` only; ``producers`` is the unfused formula (the fallback for other
dtypes and the reference for tests).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .rwkv7 import HEAD_SIZE, generalized_delta_rule, _keep_limit_bytes

W_SCALE = -math.exp(-0.5)


def producers(w_pre: torch.Tensor, kk_pre: torch.Tensor, a_pre: torch.Tensor):
    """``(w, a, b)`` from the pre-activations, computed in float32 and rounded to the input dtype."""
    dt = w_pre.dtype
    w = (W_SCALE * torch.sigmoid(w_pre.float())).to(dt)
    kk = torch.nn.functional.normalize(kk_pre.float(), dim=-1, eps=1e-12)
    return w, (-kk).to(dt), (kk * torch.sigmoid(a_pre.float())).to(dt)


@torch.library.custom_op("rwkv_ops_b200::rwkv7_fused_fwd", mutates_args=())
def _fused_fwd(r: torch.Tensor, w_pre: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kk_pre: torch.Tensor,
               a_pre: torch.Tensor, h0: Optional[torch.Tensor], keep: bool
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w_pre, k, v, kk_pre, a_pre, h0)
    B, T, H, K = r.shape
    o = torch.empty_like(r)
    ht = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    flags = _lib.ALGO_CHUNKED | (_lib.ALGO_KEEP if keep else 0)
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, K, _lib.BF16, flags)
        ws = torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_rwkv7_fused_fwd(r.data_ptr(), w_pre.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          kk_pre.data_ptr(), a_pre.data_ptr(), _lib.ptr(h0), n_state,
                                          o.data_ptr(), ht.data_ptr(), ws.data_ptr(), nws, B, T, H, K,
                                          _lib.BF16, int(keep), _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_fused_fwd")
        _lib.check_status("rwkv7_fused_fwd")
    return o, ht, (ws if keep else ws.new_empty((1,)))


@_fused_fwd.register_fake
def _(r, w_pre, k, v, kk_pre, a_pre, h0, keep):
    B, T, H, K = r.shape
    return (torch.empty_like(r), r.new_empty((B, H, K, K), dtype=torch.float32),
            r.new_empty((_lib.rwkv7_kept_bytes(B, T, H) if keep else 1,), dtype=torch.uint8))


# `kept` also serves as scratch for the backward kernels; the tiles the forward left in it are not changed.
@torch.library.custom_op("rwkv_ops_b200::rwkv7_fused_bwd", mutates_args=())
def _fused_bwd(r: torch.Tensor, w_pre: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kk_pre: torch.Tensor,
               a_pre: torch.Tensor, h0: Optional[torch.Tensor], d_o: torch.Tensor, d_ht: Optional[torch.Tensor],
               kept: torch.Tensor
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                          torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w_pre, k, v, kk_pre, a_pre, h0, d_o, d_ht, kept)
    B, T, H, K = r.shape
    dr, dw, dk, dv, du, dq = (torch.empty_like(r) for _ in range(6))
    dh0 = torch.empty(B, H, K, K, dtype=torch.float32, device=dev)
    n_state = 0 if h0 is None else h0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_rwkv7_bwd_workspace_bytes(B, T, H, K, _lib.BF16, _lib.ALGO_CHUNKED)
        have = kept.numel() >= nws
        ws = kept if have else torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_rwkv7_fused_bwd(r.data_ptr(), w_pre.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          kk_pre.data_ptr(), a_pre.data_ptr(), _lib.ptr(h0), n_state,
                                          d_o.data_ptr(), _lib.ptr(d_ht), dr.data_ptr(), dw.data_ptr(),
                                          dk.data_ptr(), dv.data_ptr(), du.data_ptr(), dq.data_ptr(),
                                          dh0.data_ptr(), ws.data_ptr(), nws, B, T, H, K, _lib.BF16, int(have),
                                          _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_fused_bwd")
        _lib.check_status("rwkv7_fused_bwd")
    return dr, dw, dk, dv, du, dq, dh0


@_fused_bwd.register_fake
def _(r, w_pre, k, v, kk_pre, a_pre, h0, d_o, d_ht, kept):
    B, T, H, K = r.shape
    e = torch.empty_like
    return e(r), e(r), e(r), e(r), e(r), e(r), r.new_empty((B, H, K, K), dtype=torch.float32)


def _setup_ctx(ctx, inputs, output):
    r, w_pre, k, v, kk_pre, a_pre, h0, keep = inputs
    ctx.save_for_backward(r, w_pre, k, v, kk_pre, a_pre, h0, output[2])
    ctx.set_materialize_grads(False)


def _backward(ctx, d_o, d_ht, d_kept):
    r, w_pre, k, v, kk_pre, a_pre, h0, kept = ctx.saved_tensors
    if d_o is None:
        d_o = torch.zeros_like(r)
    d_o = d_o.to(r.dtype).contiguous()
    if d_ht is not None:
        d_ht = d_ht.to(torch.float32).contiguous()
    dr, dw, dk, dv, du, dq, dh0 = _fused_bwd(r, w_pre, k, v, kk_pre, a_pre, h0, d_o, d_ht, kept)
    if h0 is None or not ctx.needs_input_grad[6]:
        dh0 = None
    elif h0.shape[0] == 1 and dh0.shape[0] != 1:
        dh0 = dh0.sum(0, keepdim=True)
    return dr, dw, dk, dv, du, dq, dh0, None


torch.library.register_autograd("rwkv_ops_b200::rwkv7_fused_fwd", _backward, setup_context=_setup_ctx)


def generalized_delta_rule_fused(r, w_pre, k, v, kk_pre, a_pre, initial_state=None, output_final_state=True):
    """``generalized_delta_rule(r, w, k, v, a, b)`` with ``(w, a, b) = producers(w_pre, kk_pre, a_pre)``
    computed inside the operator (see the module docstring).  ``[B, T, H, 64]`` tensors; returns
    ``(o, final_state)`` or just ``o``."""
    _lib.require_cuda(r, w_pre, k, v, kk_pre, a_pre, initial_state)
    if r.dim() != 4 or r.shape[-1] != HEAD_SIZE:
        raise ValueError(f"expected 4-D token tensors with head size {HEAD_SIZE}, got {tuple(r.shape)}")
    for name, x in (("w_pre", w_pre), ("k", k), ("v", v), ("kk_pre", kk_pre), ("a_pre", a_pre)):
        if x.shape != r.shape:
            raise ValueError(f"{name} has shape {tuple(x.shape)}, expected {tuple(r.shape)}")
    B, T, H = r.shape[0], r.shape[1], r.shape[2]
    if r.dtype != torch.bfloat16 or T == 1 or any(x.dtype != r.dtype for x in (w_pre, k, v, kk_pre, a_pre)):
        w, a, b = producers(w_pre, kk_pre, a_pre)      # unfused: other dtypes and single-token steps
        return generalized_delta_rule(r, w, k, v, a, b, initial_state=initial_state,
                                      output_final_state=output_final_state)
    h0 = None
    if initial_state is not None:
        if initial_state.dim() != 4 or tuple(initial_state.shape[1:]) != (H, HEAD_SIZE, HEAD_SIZE) \
                or initial_state.shape[0] not in (1, B):
            raise ValueError(
                f"initial_state must be [B or 1, {H}, {HEAD_SIZE}, {HEAD_SIZE}], got {tuple(initial_state.shape)}")
        h0 = initial_state.to(torch.float32).contiguous()
    args = [x.contiguous() for x in (r, w_pre, k, v, kk_pre, a_pre)]
    needs_grad = torch.is_grad_enabled() and (
        any(x.requires_grad for x in args) or (h0 is not None and h0.requires_grad))
    keep = False
    if needs_grad:
        nws = _lib.load().rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, HEAD_SIZE, _lib.BF16,
                                                              _lib.ALGO_CHUNKED | _lib.ALGO_KEEP)
        keep = nws <= _keep_limit_bytes(r.device)
    o, ht, _ = _fused_fwd(*args, h0, keep)
    return (o, ht) if output_final_state else o
