"""RWKV6 wkv operator: the reference's ``RWKVKernelOperator`` interface over the CUDA library.

Mirrors ``get_rwkv6_kernel`` / ``RWKVKernelOperator`` of the reference
(``rwkv_ops/rwkv6_kernel/__init__.py:9-96``, ``rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:5-86``,
``rwkv_ops/rwkv6_kernel/torch_rwkv_kernel.py:50-304``): constructor ``(head_size,
max_sequence_length, ops_loop=False)`` and call ``(r, k, v, w, u, with_state=False,
init_state=None, state_map=None) -> (y, state | None)``.  Unlike the reference's GPU operator,
gradients flow with ``with_state=True`` (to ``init_state`` as well), ``state_map`` works, and
``max_sequence_length`` is not a compile-time constant (it is accepted and ignored).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _lib

HEAD_SIZE = 64                  # the head size of the chunked tensor-core path
HEAD_SIZES = (32, 64, 128)      # 32 and 128 run the float32 recurrence
_ALGO_NAMES = {"auto": _lib.ALGO_AUTO, "recurrent": _lib.ALGO_RECURRENT, "chunked": _lib.ALGO_CHUNKED}


def _default_algo() -> int:
    return _ALGO_NAMES[os.environ.get("RWKV_OPS_B200_WKV6_ALGO", "auto").lower()]


@torch.library.custom_op("rwkv_ops_b200::wkv6_fwd", mutates_args=())
def _wkv6_fwd(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
              s0: Optional[torch.Tensor], state_map: Optional[torch.Tensor], algo: int, keep: bool
              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, k, v, w, u, s0, state_map)
    B, T, C = r.shape
    H, N = u.shape                      # u arrives as [H, head_size]
    code = _lib.dtype_code(r.dtype)
    y = torch.empty_like(r)
    sT = torch.empty(B, H, N, N, dtype=torch.float32, device=dev)
    n_state = 0 if s0 is None else s0.shape[0]
    with torch.cuda.device(dev):
        # a training forward of the chunked path leaves the chunk-boundary states for the backward; an
        # inference forward needs a few bytes per (batch, head) for the decay-range marks
        flags = algo | (_lib.ALGO_KEEP if keep else 0)
        nws = lib.rwkvb200_wkv6_fwd_workspace_bytes(B, T, H, N, code, flags)
        kept = torch.empty(nws, dtype=torch.uint8, device=dev)
        rc = lib.rwkvb200_wkv6_fwd(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                   _lib.ptr(s0), n_state, _lib.ptr(state_map), y.data_ptr(), sT.data_ptr(),
                                   kept.data_ptr() if nws else None, nws,
                                   B, T, H, N, code, flags, _lib.stream_ptr(dev))
        _lib.check(rc, "wkv6_fwd")
        _lib.check_status("wkv6_fwd")
    if not keep:
        kept = kept.new_empty(0)
    return y, sT, kept


@_wkv6_fwd.register_fake
def _(r, k, v, w, u, s0, state_map, algo, keep):
    B, T, C = r.shape
    H, N = u.shape
    chunked = (algo & 0xff) != _lib.ALGO_RECURRENT and N == HEAD_SIZE
    return (torch.empty_like(r), r.new_empty((B, H, N, N), dtype=torch.float32),
            r.new_empty((_lib.wkv6_kept_bytes(B, T, H) if keep and chunked else 0,), dtype=torch.uint8))


# `kept` (the forward's chunk-boundary states) also holds the backward's scratch rows; what the forward
# left there is not changed, so the op declares no mutation (a second backward through the graph stays legal).
@torch.library.custom_op("rwkv_ops_b200::wkv6_bwd", mutates_args=())
def _wkv6_bwd(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
              s0: Optional[torch.Tensor], state_map: Optional[torch.Tensor],
              d_y: torch.Tensor, d_sT: Optional[torch.Tensor], kept: torch.Tensor, algo: int
              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = _lib.require_cuda(r, k, v, w, u, s0, state_map, d_y, d_sT)
    B, T, C = r.shape
    H, N = u.shape
    code = _lib.dtype_code(r.dtype)
    dr, dk, dv, dw = (torch.empty_like(r) for _ in range(4))
    du = torch.empty(H, N, dtype=torch.float32, device=dev)
    ds0 = torch.empty(B, H, N, N, dtype=torch.float32, device=dev)
    n_state = 0 if s0 is None else s0.shape[0]
    with torch.cuda.device(dev):
        nws = lib.rwkvb200_wkv6_bwd_workspace_bytes(B, T, H, N, code, algo)
        have = kept.numel() >= nws and kept.numel() > 0      # the forward left its chunk-boundary states
        ws = kept if have else torch.empty(nws, dtype=torch.uint8, device=dev)
        algo = algo | (_lib.ALGO_KEEP if have else 0)
        rc = lib.rwkvb200_wkv6_bwd(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(),
                                   _lib.ptr(s0), n_state, _lib.ptr(state_map), d_y.data_ptr(), _lib.ptr(d_sT),
                                   dr.data_ptr(), dk.data_ptr(), dv.data_ptr(), dw.data_ptr(), du.data_ptr(),
                                   ds0.data_ptr(), ws.data_ptr(), nws, B, T, H, N, code, algo,
                                   _lib.stream_ptr(dev))
        _lib.check(rc, "wkv6_bwd")
        _lib.check_status("wkv6_bwd")
    return dr, dk, dv, dw, du, ds0


@_wkv6_bwd.register_fake
def _(r, k, v, w, u, s0, state_map, d_y, d_sT, kept, algo):
    B, T, C = r.shape
    H, N = u.shape
    e = torch.empty_like
    return (e(r), e(r), e(r), e(r), r.new_empty((H, N), dtype=torch.float32),
            r.new_empty((B, H, N, N), dtype=torch.float32))


def _setup_ctx(ctx, inputs, output):
    r, k, v, w, u, s0, state_map, algo, keep = inputs
    ctx.save_for_backward(r, k, v, w, u, s0, state_map, output[2])
    ctx.set_materialize_grads(False)
    ctx.algo = algo


def _backward(ctx, d_y, d_sT, d_kept):
    r, k, v, w, u, s0, state_map, kept = ctx.saved_tensors
    if d_y is None:
        d_y = torch.zeros_like(r)
    d_y = d_y.to(r.dtype).contiguous()
    if d_sT is not None:
        d_sT = d_sT.to(torch.float32).contiguous()
    dr, dk, dv, dw, du, ds0_rows = _wkv6_bwd(r, k, v, w, u, s0, state_map, d_y, d_sT, kept, ctx.algo)
    ds0 = None
    if s0 is not None and ctx.needs_input_grad[5]:
        n_state, B = s0.shape[0], r.shape[0]
        if state_map is not None:
            idx = state_map.to(torch.int64)
        elif n_state == 1:
            idx = torch.zeros(B, dtype=torch.int64, device=r.device)
        else:
            idx = torch.arange(B, device=r.device)
        # several batch rows may start from the same table row: their gradients add up
        ds0 = torch.zeros_like(s0).index_add_(0, idx, ds0_rows)
    return dr, dk, dv, dw, du, ds0, None, None, None


torch.library.register_autograd("rwkv_ops_b200::wkv6_fwd", _backward, setup_context=_setup_ctx)


class RWKVKernelOperator:
    """Drop-in for the class returned by the reference's ``get_rwkv6_kernel``."""

    def __init__(self, head_size, max_sequence_length, ops_loop=False):
        if head_size not in HEAD_SIZES:
            raise ValueError(f"rwkv_ops_b200 wkv6 supports head sizes {HEAD_SIZES}, got {head_size}")
        self.head_size = head_size
        self.max_sequence_length = max_sequence_length   # kept for compatibility; no limit applies
        self.ops_loop = ops_loop

    def __call__(self, r, k, v, w, u, with_state=False, init_state=None, state_map=None):
        dev = _lib.require_cuda(r, k, v, w, u, init_state)
        if r.dim() != 3:
            raise ValueError(f"expected [B, T, C] tensors, got {tuple(r.shape)}")
        B, T, C = r.shape
        N = self.head_size
        assert C % N == 0, "hidden size must be a multiple of head_size"
        H = C // N
        for name, x in (("k", k), ("v", v), ("w", w)):
            assert x.shape == r.shape, f"{name} has shape {tuple(x.shape)}, expected {tuple(r.shape)}"
            assert x.dtype == r.dtype, "r, k, v, w must share one dtype"
        assert u.numel() == C, f"u must have {C} elements"
        dt = r.dtype
        cdt = dt if dt in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        state_dtype = torch.float32 if dt == torch.float16 else dt

        s0 = None
        smap = None
        if init_state is not None:
            assert init_state.dim() in (3, 4), "init_state must be [n_state, H, N, N] or [H, N, N]"
            if init_state.dim() == 3:
                assert tuple(init_state.shape) == (H, N, N), "init_state must be [H, N, N]"
                init_state = init_state[None]
            else:
                assert tuple(init_state.shape[1:]) == (H, N, N), "init_state must be [n_state, H, N, N]"
            n_state = init_state.shape[0]
            if state_map is None:
                if n_state not in (1, B):
                    raise ValueError("state_map cannot be inferred from init_state; pass it explicitly")
            else:
                if isinstance(state_map, (list, tuple)):
                    state_map = torch.tensor(state_map, dtype=torch.int32)
                assert state_map.dtype in (torch.int32, torch.int64), "state_map must be int32 or int64"
                assert state_map.numel() == B, "state_map must have one entry per batch row"
                if not state_map.is_cuda:
                    # a host-side map (list, CPU tensor) is range-checked here, where the reference
                    # device-asserts (rwkv6_kernel/torch_kernel/wkv6_cuda.cu:81); a map that already lives
                    # on the device is not read back (that would stall the stream on every call): the
                    # kernels clamp its entries to the table instead of trapping
                    assert bool((state_map >= 0).all()) and bool((state_map < n_state).all()), (
                        f"state_map values must lie in [0, {n_state})")
                smap = state_map.to(device=dev, dtype=torch.int32).contiguous().view(B)
            s0 = init_state.to(torch.float32).contiguous()
        else:
            assert state_map is None, "state_map needs init_state"

        algo = _default_algo()
        if N != HEAD_SIZE:
            if algo == _lib.ALGO_CHUNKED:
                raise ValueError("the chunked wkv6 path is built for head size 64")
            algo = _lib.ALGO_RECURRENT
        needs_grad = torch.is_grad_enabled() and (
            any(x.requires_grad for x in (r, k, v, w, u)) or (init_state is not None and init_state.requires_grad))
        keep = needs_grad and algo != _lib.ALGO_RECURRENT and T > 1
        y, sT, _ = _wkv6_fwd(r.to(cdt).contiguous(), k.to(cdt).contiguous(), v.to(cdt).contiguous(),
                             w.to(cdt).contiguous(), u.reshape(H, N).to(torch.float32).contiguous(), s0, smap,
                             algo, keep)
        if y.dtype != dt:
            y = y.to(dt)
        if with_state:
            return y, sT.to(state_dtype)
        return y, None


def get_rwkv6_kernel(KERNEL_TYPE: str = "cuda"):
    """Reference signature (``rwkv_ops/rwkv6_kernel/__init__.py:9``); ``KERNEL_TYPE`` is ignored."""
    return RWKVKernelOperator
