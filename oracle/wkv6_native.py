"""CPU restatement of the reference's native RWKV6 wkv operator.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows ``rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:5-86`` of the reference:

* ``r, k, v, w`` are ``[B, T, C]`` with ``C = H * head_size``; ``u`` is anything
  with ``C`` elements (``:16-21``);
* ``init_state`` is ``[n_state, H, N, N]`` or ``[H, N, N]``, key index first;
  ``state_map`` picks one initial state per batch row and defaults to zeros for
  one state, to ``arange(B)`` for ``B`` states and is an error otherwise
  (``:23-57``);
* the decay is ``exp(-exp(w))`` (``:63``);
* one token does ``y = r^T (diag(u) k v^T + S)`` with the *previous* state and
  then ``S <- diag(d) S + k v^T`` (``:68-77``);
* returns ``(y, S)`` when ``with_state`` else ``(y, None)`` (``:84-86``).

The output is written in place instead of through ``slice_update``; results are
identical.  ``compute_dtype=torch.float64`` gives the high-precision variant.
"""
from __future__ import annotations

import torch


class RWKVKernelOperator:
    def __init__(self, head_size, max_sequence_length, compute_dtype=None):
        self.head_size = head_size
        self.max_sequence_length = max_sequence_length
        self.compute_dtype = compute_dtype

    def __call__(self, r, k, v, w, u, with_state=False, init_state=None, state_map=None):
        B, T, C = r.shape
        N = self.head_size
        assert C % N == 0
        H = C // N
        cd = self.compute_dtype or r.dtype
        out_dtype = r.dtype
        w_ = w.to(cd).reshape(B, T, H, N, 1)
        k_ = k.to(cd).reshape(B, T, H, N, 1)
        v_ = v.to(cd).reshape(B, T, H, 1, N)
        r_ = r.to(cd).reshape(B, T, H, 1, N)
        u_ = u.to(cd).reshape(1, H, N, 1)

        if init_state is not None:
            assert init_state.dim() in (3, 4), "init_state must be [n_state, H, N, N] or [H, N, N]"
            if init_state.dim() == 3:
                assert tuple(init_state.shape) == (H, N, N)
                init_state = init_state[None]
            else:
                assert tuple(init_state.shape[1:]) == (H, N, N)
            n_state = init_state.shape[0]
            if state_map is None:
                if n_state == 1:
                    state_map = torch.zeros(B, dtype=torch.int32)
                elif n_state == B:
                    state_map = torch.arange(B, dtype=torch.int32)
                else:
                    raise ValueError("state_map cannot be inferred from init_state; pass it explicitly")
            else:
                if isinstance(state_map, list):
                    state_map = torch.tensor(state_map, dtype=torch.int32)
                state_map = state_map.to(torch.int32)
                assert bool((state_map >= 0).all()) and bool((state_map < n_state).all()), (
                    f"state_map values must lie in [0, {n_state})"
                )
            s = init_state.to(cd).index_select(0, state_map.to(torch.int64))
        else:
            assert state_map is None
            s = torch.zeros(B, H, N, N, dtype=cd)

        decay = torch.exp(-torch.exp(w_))
        track = any(x.requires_grad for x in (r, k, v, w, u)) or (
            init_state is not None and init_state.requires_grad
        )
        ys = [] if track else torch.empty(B, T, C, dtype=cd)
        for t in range(T):
            kv = k_[:, t] @ v_[:, t]                        # [B,H,K,V]
            y_t = (r_[:, t] @ (u_ * kv + s)).reshape(B, C)  # [B,H,1,V] -> [B,C]
            s = kv + decay[:, t] * s
            if track:
                ys.append(y_t)
            else:
                ys[:, t] = y_t
        y = torch.stack(ys, dim=1) if track else ys
        y = y.to(out_dtype)
        if with_state:
            return y, s
        return y, None


def wkv6_manual_backward(r, k, v, w, u, s0, d_y, d_final_state, head_size,
                         compute_dtype: torch.dtype = torch.float64):
    """Hand-derived reverse recurrence for wkv6 (no autograd).

    ``s0`` is the per-batch initial state ``[B, H, K, V]`` (already gathered
    through ``state_map``) or None.  Returns ``(dr, dk, dv, dw, du, ds0)`` with
    ``du`` of shape ``[H, N]`` and ``ds0`` per batch row; a caller with repeated
    ``state_map`` entries sums ``ds0`` rows itself.
    """
    cd = compute_dtype
    B, T, C = r.shape
    N = head_size
    H = C // N
    r_ = r.to(cd).reshape(B, T, H, N); k_ = k.to(cd).reshape(B, T, H, N)
    v_ = v.to(cd).reshape(B, T, H, N); w_ = w.to(cd).reshape(B, T, H, N)
    dy = d_y.to(cd).reshape(B, T, H, N)
    u_ = u.to(cd).reshape(H, N)
    ew = torch.exp(w_)
    decay = torch.exp(-ew)
    S = torch.zeros(B, H, N, N, dtype=cd) if s0 is None else s0.to(cd).clone()
    states = [S]
    for t in range(T):
        S = decay[:, t].unsqueeze(-1) * S + k_[:, t].unsqueeze(-1) * v_[:, t].unsqueeze(-2)
        states.append(S)
    G = torch.zeros(B, H, N, N, dtype=cd) if d_final_state is None else d_final_state.to(cd).clone()
    dr = torch.empty_like(r_); dk = torch.empty_like(r_); dv = torch.empty_like(r_); dw = torch.empty_like(r_)
    du = torch.zeros(H, N, dtype=cd)
    for t in range(T - 1, -1, -1):
        S_p = states[t]
        rt, kt, vt, dyt = r_[:, t], k_[:, t], v_[:, t], dy[:, t]
        dyv = (dyt * vt).sum(-1, keepdim=True)               # [B,H,1]  sum_v dy v
        dr[:, t] = u_ * kt * dyv + (S_p * dyt.unsqueeze(-2)).sum(-1)
        du += (rt * kt * dyv).sum(0)
        dk[:, t] = rt * u_ * dyv + (G * vt.unsqueeze(-2)).sum(-1)
        ruk = (rt * u_ * kt).sum(-1, keepdim=True)           # [B,H,1]
        dv[:, t] = dyt * ruk + (G * kt.unsqueeze(-1)).sum(-2)
        dd = (G * S_p).sum(-1)
        dw[:, t] = dd * decay[:, t] * (-ew[:, t])
        G = decay[:, t].unsqueeze(-1) * G + rt.unsqueeze(-1) * dyt.unsqueeze(-2)
    return (dr.reshape(B, T, C), dk.reshape(B, T, C), dv.reshape(B, T, C), dw.reshape(B, T, C), du, G)
