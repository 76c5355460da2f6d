"""CPU restatement of the reference's native RWKV7 generalized delta rule.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows ``rwkv_ops/rwkv7_kernel/native_keras_op.py:23-95`` of the reference:

* inputs are cast to float32 (``:16``), the decay is ``exp(-exp(w))`` (``:58``);
* the state is ``[B, H, V, K]`` (value index first), zero or ``initial_state``,
  and an ``initial_state`` with a leading dimension of 1 is broadcast over the
  batch (``:60-65``);
* one token does ``S <- S * d[None, :] + (S a) b^T + v k^T`` and then
  ``o = S r`` with the *updated* state (``:80-91``);
* the output is cast back to ``r``'s dtype and the state is returned only when
  ``output_final_state`` is true (``:93-95``).

Differences from the reference file, none of which changes a result: the output
is written in place instead of through a whole-tensor ``slice_update`` (the
reference's copy makes its cost quadratic in T), and ``head_first=True`` means
``[B, H, T, .]`` tensors in and out, which is what the reference's GPU path does
(``rwkv_ops/rwkv7_kernel/torch_op.py:451-455,486``); the native file reads the
shape before transposing (``native_keras_op.py:49-50``) and is not usable for it.

``compute_dtype=torch.float64`` gives the high-precision variant used to judge
which of two float32 results is closer to the truth.
"""
from __future__ import annotations

import torch


def generalized_delta_rule(
    r,
    w,
    k,
    v,
    a,
    b,
    initial_state=None,
    output_final_state: bool = True,
    head_first: bool = False,
    compute_dtype: torch.dtype = torch.float32,
):
    out_dtype = r.dtype
    cd = compute_dtype

    def prep(x):
        x = x.to(cd)
        return x.permute(0, 2, 1, 3) if head_first else x

    r_, w_, k_, v_, a_, b_ = (prep(x) for x in (r, w, k, v, a, b))
    B, T, H, N = r_.shape
    decay = torch.exp(-torch.exp(w_))
    if initial_state is not None:
        state = initial_state.to(cd)
        if state.shape[0] == 1:
            state = state.broadcast_to(B, H, N, N)
    else:
        state = torch.zeros(B, H, N, N, dtype=cd)
    track = any(x.requires_grad for x in (r, w, k, v, a, b)) or (
        initial_state is not None and initial_state.requires_grad
    )
    outs = [] if track else torch.empty(B, T, H, N, dtype=cd)
    for t in range(T):
        kk = k_[:, t].unsqueeze(-2)  # [B,H,1,K]
        rr = r_[:, t].unsqueeze(-1)  # [B,H,K,1]
        vv = v_[:, t].unsqueeze(-1)  # [B,H,V,1]
        aa = a_[:, t].unsqueeze(-1)  # [B,H,K,1]
        bb = b_[:, t].unsqueeze(-2)  # [B,H,1,K]
        state = state * decay[:, t].unsqueeze(-2) + (state @ aa) @ bb + vv @ kk
        o_t = (state @ rr).squeeze(-1)  # [B,H,V]
        if track:
            outs.append(o_t)
        else:
            outs[:, t] = o_t
    out = torch.stack(outs, dim=1) if track else outs
    if head_first:
        out = out.permute(0, 2, 1, 3)
    out = out.to(out_dtype)
    if output_final_state:
        return out, state
    return out


def rwkv7_manual_backward(r, w, k, v, a, b, initial_state, d_out, d_final_state,
                          compute_dtype: torch.dtype = torch.float64):
    """Hand-derived reverse recurrence (no autograd), ``[B,T,H,.]`` layout only.

    Independent of autograd so that the two can be checked against each other,
    and cheap enough in memory to run a few (batch, head) units at full length.
    Returns ``(dr, dw, dk, dv, da, db, d_initial_state)`` in ``compute_dtype``.
    ``d_final_state`` may be None.  State tensors are ``[B, H, V, K]``.
    """
    cd = compute_dtype
    r_, w_, k_, v_, a_, b_, do = (x.to(cd) for x in (r, w, k, v, a, b, d_out))
    B, T, H, N = r_.shape
    ew = torch.exp(w_)
    decay = torch.exp(-ew)
    S = torch.zeros(B, H, N, N, dtype=cd) if initial_state is None else initial_state.to(cd).broadcast_to(B, H, N, N).clone()
    states = [S]
    for t in range(T):
        sa = S @ a_[:, t].unsqueeze(-1)
        S = S * decay[:, t].unsqueeze(-2) + sa @ b_[:, t].unsqueeze(-2) + v_[:, t].unsqueeze(-1) @ k_[:, t].unsqueeze(-2)
        states.append(S)
    dS = torch.zeros(B, H, N, N, dtype=cd) if d_final_state is None else d_final_state.to(cd).clone()
    dr = torch.empty_like(r_); dw = torch.empty_like(r_); dk = torch.empty_like(r_)
    dv = torch.empty_like(r_); da = torch.empty_like(r_); db = torch.empty_like(r_)
    for t in range(T - 1, -1, -1):
        S_t, S_p = states[t + 1], states[t]
        do_t = do[:, t].unsqueeze(-1)                      # [B,H,V,1]
        dr[:, t] = (S_t.transpose(-1, -2) @ do_t).squeeze(-1)
        dS = dS + do_t @ r_[:, t].unsqueeze(-2)
        sa = S_p @ a_[:, t].unsqueeze(-1)                  # [B,H,V,1]
        dv[:, t] = (dS @ k_[:, t].unsqueeze(-1)).squeeze(-1)
        dk[:, t] = (dS.transpose(-1, -2) @ v_[:, t].unsqueeze(-1)).squeeze(-1)
        dsa = dS @ b_[:, t].unsqueeze(-1)                  # [B,H,V,1]
        db[:, t] = (dS.transpose(-1, -2) @ sa).squeeze(-1)
        dd = (dS * S_p).sum(dim=-2)                        # [B,H,K]
        da[:, t] = (S_p.transpose(-1, -2) @ dsa).squeeze(-1)
        dw[:, t] = dd * decay[:, t] * (-ew[:, t])
        dS = dS * decay[:, t].unsqueeze(-2) + dsa @ a_[:, t].unsqueeze(-2)
    return dr, dw, dk, dv, da, db, dS
