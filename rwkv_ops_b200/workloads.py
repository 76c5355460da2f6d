"""Seeded synthetic inputs with the value distributions of the benchmark configurations.

The reference measures on no dataset; every workload here is synthetic and is
reproducible from its seed.  Shapes follow the reference operators' contracts:
RWKV7 tensors are ``[B, T, H, 64]`` (``rwkv_ops/rwkv7_kernel/native_keras_op.py:49``)
and RWKV6 tensors are ``[B, T, C]`` (``rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py:13``).
"""
from __future__ import annotations

import torch

W_SCALE = -0.606531  # the RWKV7 time-mix bounds w to (-0.606531, 0) before exp(-exp(w))


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def rwkv7_inputs(B, T, H, K=64, *, dtype=torch.float32, seed=1000, device="cpu",
                 with_state=False, n_state=None, with_grads=False):
    """r,k,v ~ N(0,1); kk = unit-norm N(0,1); a = -kk; b = kk*sigmoid(N(0,1));
    w = -0.606531*sigmoid(N(0,1)); state ~ N(0, 0.1^2) as [n_state, H, 64, 64] float32.

    Values are drawn in float32 and then rounded to ``dtype``; an oracle run sees
    the rounded values.  Returns a dict; gradient seeds ``d_out ~ N(0,1)`` and
    ``d_state ~ N(0, 0.1^2)`` are included when ``with_grads``.
    """
    g = _gen(seed, device)
    shp = (B, T, H, K)

    def n(*s):
        return torch.randn(*s, generator=g, device=device, dtype=torch.float32)

    r, k, v = n(*shp), n(*shp), n(*shp)
    kk = torch.nn.functional.normalize(n(*shp), dim=-1)
    a = -kk
    b = kk * torch.sigmoid(n(*shp))
    w = W_SCALE * torch.sigmoid(n(*shp))
    out = {x: t.to(dtype) for x, t in dict(r=r, w=w, k=k, v=v, a=a, b=b).items()}
    if with_state:
        out["initial_state"] = 0.1 * n(n_state or B, H, K, K)
    if with_grads:
        out["d_out"] = n(*shp).to(dtype)
        out["d_state"] = 0.1 * n(B, H, K, K)
    return out


def rwkv7_pad_lengths(B, T, max_pad=512, seed=1002):
    """Per-sequence valid lengths ``T - U{0..max_pad}`` (config 2's trailing padding)."""
    g = torch.Generator().manual_seed(seed)
    pad = torch.randint(0, min(max_pad, T - 1) + 1, (B,), generator=g)
    return T - pad


def apply_w_padding(w, lengths):
    """The reference's padding recipe: ``w += (1 - mask) * -1e9`` on the padded
    tail (``README.md:92-98``), which turns the decay into exactly 1 there."""
    B, T = w.shape[:2]
    pos = torch.arange(T, device=w.device)[None, :]
    mask = (pos < lengths.to(w.device)[:, None]).to(torch.float32)
    return (w.float() + (1.0 - mask)[:, :, None, None] * -1e9).to(w.dtype)


def wkv6_inputs(B, T, H, N=64, *, dtype=torch.float32, seed=1004, device="cpu",
                n_state=None, with_grads=False):
    """r,k,v ~ N(0,1); w = -exp(N(-0.5, 0.5^2)); u ~ N(0, 0.1^2) [H,N];
    init_state ~ N(0, 0.1^2) [n_state,H,N,N]; state_map ~ U{0..n_state-1} int32 [B]."""
    g = _gen(seed, device)
    C = H * N

    def n(*s):
        return torch.randn(*s, generator=g, device=device, dtype=torch.float32)

    r, k, v = n(B, T, C), n(B, T, C), n(B, T, C)
    w = -torch.exp(-0.5 + 0.5 * n(B, T, C))
    u = 0.1 * n(H, N)
    out = {x: t.to(dtype) for x, t in dict(r=r, k=k, v=v, w=w, u=u).items()}
    if n_state:
        out["init_state"] = (0.1 * n(n_state, H, N, N)).to(dtype)
        out["state_map"] = torch.randint(0, n_state, (B,), generator=g, device=device, dtype=torch.int32)
    if with_grads:
        out["d_y"] = n(B, T, C).to(dtype)
        out["d_state"] = (0.1 * n(B, H, N, N)).to(dtype)
    return out


def rel_l2(x, ref):
    """``||x - ref||_2 / ||ref||_2`` in float64, the parity metric of every test."""
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = ref.norm()
    return float((x - ref).norm() / den) if den > 0 else float((x - ref).norm())
