"""Token-by-token RWKV7 decoding with the state kept in place on the device.

The reference decodes by calling ``generalized_delta_rule`` with ``T == 1`` and feeding
``final_state`` back as ``initial_state`` (``rwkv_ops/rwkv7_kernel/native_keras_op.py:60-95``): every
step allocates and returns a new ``[B, H, 64, 64]`` float32 state.  ``Rwkv7DecodeState`` owns one
state buffer, updates it in place with one kernel launch per token and nothing else on the stream
(no allocation besides the 64-value output rows), and can hold the state in bfloat16, which halves
the bytes a step moves.  The float32 mode computes exactly what the ``T == 1`` operator computes.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

HEAD_SIZE = 64


@torch.library.custom_op("rwkv_ops_b200::rwkv7_decode_step", mutates_args=("state",))
def _decode_step(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
                 b: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    dev = _lib.require_cuda(r, w, k, v, a, b, state)
    B, H = state.shape[0], state.shape[1]
    o = torch.empty_like(r)
    with torch.cuda.device(dev):
        rc = lib.rwkvb200_rwkv7_decode_step(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                            b.data_ptr(), state.data_ptr(), _lib.dtype_code(state.dtype),
                                            o.data_ptr(), B, H, HEAD_SIZE, _lib.dtype_code(r.dtype),
                                            _lib.stream_ptr(dev))
        _lib.check(rc, "rwkv7_decode_step")
    return o


@_decode_step.register_fake
def _(r, w, k, v, a, b, state):
    return torch.empty_like(r)


class Rwkv7DecodeState:
    """State of ``B`` sequences x ``H`` heads for single-token steps.

    ``state`` is ``[B, H, 64, 64]`` (value index before key index, the layout of the operator's
    ``final_state``), float32 or bfloat16.  ``step`` takes the six token tensors as ``[B, 1, H, 64]``
    (the operator's layout with ``T == 1``) or ``[B, H, 64]`` and returns ``o`` in the same shape.
    """

    def __init__(self, batch: int, heads: int, *, state_dtype: torch.dtype = torch.float32, device="cuda",
                 initial_state: Optional[torch.Tensor] = None):
        if state_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("state_dtype must be float32 or bfloat16")
        shape = (batch, heads, HEAD_SIZE, HEAD_SIZE)
        if initial_state is not None:
            _lib.require_cuda(initial_state)
            if initial_state.dim() != 4 or tuple(initial_state.shape[1:]) != shape[1:] \
                    or initial_state.shape[0] not in (1, batch):
                raise ValueError(f"initial_state must be [{batch} or 1, {heads}, 64, 64], got {tuple(initial_state.shape)}")
            self.state = initial_state.expand(shape).to(state_dtype).contiguous().clone()
        else:
            self.state = torch.zeros(shape, dtype=state_dtype, device=device)
        if not self.state.is_cuda:
            raise _lib.RwkvB200Error("Rwkv7DecodeState lives on a CUDA device; there is no CPU fallback.")

    @torch.no_grad()
    def step(self, r, w, k, v, a, b):
        shape = r.shape
        B, H = self.state.shape[0], self.state.shape[1]
        if tuple(shape) not in ((B, 1, H, HEAD_SIZE), (B, H, HEAD_SIZE)):
            raise ValueError(f"expected token tensors [{B}, 1, {H}, 64] or [{B}, {H}, 64], got {tuple(shape)}")
        dt = r.dtype if r.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        args = []
        for name, x in (("r", r), ("w", w), ("k", k), ("v", v), ("a", a), ("b", b)):
            if x.shape != shape:
                raise ValueError(f"{name} has shape {tuple(x.shape)}, expected {tuple(shape)}")
            args.append(x.to(dt).contiguous().view(B, H, HEAD_SIZE))
        o = _decode_step(*args, self.state)
        return o.view(shape).to(r.dtype)

    def final_state(self) -> torch.Tensor:
        """The state as the operator would return it (float32 copy)."""
        return self.state.to(torch.float32)
