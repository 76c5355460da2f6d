"""Generate the golden fixtures in this folder from the reference's own native operators.

Run where the reference checkout is available (it is not needed to *use* the fixtures):

    python tests/golden/make_golden.py --reference /path/to/rwkv_ops_checkout

The two native operator files of the reference
(``rwkv_ops/rwkv7_kernel/native_keras_op.py`` and
``rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py``) are loaded unmodified through
``oracle.keras_shim`` (keras itself cannot be installed offline) and evaluated on
seeded inputs in float32 on CPU.  Gradients come from torch autograd through that
same unmodified code.  Each fixture stores inputs and outputs, so reading one
needs neither the reference nor a particular random-number generator.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import keras_shim  # noqa: E402
from rwkv_ops_b200 import workloads  # noqa: E402


def _np(t):
    t = t.detach()
    if t.dtype == torch.bfloat16:
        # store the exact bf16 values as float32
        return t.float().numpy()
    return t.numpy()


def rwkv7_case(ref7, name, B, T, H, *, dtype=torch.float32, seed, state=None, grads=True):
    n_state = {None: None, "per_batch": B, "broadcast": 1}[state]
    d = workloads.rwkv7_inputs(B, T, H, dtype=dtype, seed=seed, with_state=state is not None,
                               n_state=n_state, with_grads=True)
    names = ["r", "w", "k", "v", "a", "b"]
    leaves = {n: d[n].clone().requires_grad_(grads) for n in names}
    h0 = d.get("initial_state")
    if h0 is not None:
        h0 = h0.clone().requires_grad_(grads)
    o, s = ref7.generalized_delta_rule(leaves["r"], leaves["w"], leaves["k"], leaves["v"], leaves["a"],
                                       leaves["b"], initial_state=h0, output_final_state=True)
    out = {f"in_{n}": _np(d[n]) for n in names}
    out["dtype"] = np.array(str(dtype).replace("torch.", ""))
    if h0 is not None:
        out["in_initial_state"] = _np(h0)
    out["o"] = _np(o)
    out["final_state"] = _np(s)
    if grads:
        loss = (o.float() * d["d_out"].float()).sum() + (s * d["d_state"]).sum()
        loss.backward()
        out["d_out"] = _np(d["d_out"])
        out["d_state"] = _np(d["d_state"])
        for n in names:
            out[f"grad_{n}"] = _np(leaves[n].grad)
        if h0 is not None:
            out["grad_initial_state"] = _np(h0.grad)
    np.savez_compressed(os.path.join(HERE, f"rwkv7_{name}.npz"), **out)
    print("wrote", name, {k: v.shape for k, v in out.items() if k in ("o", "final_state")})


def wkv6_case(ref6, name, B, T, H, *, seed, n_state=None, explicit_map=True, with_state=True, grads=True):
    N = 64
    d = workloads.wkv6_inputs(B, T, H, seed=seed, n_state=n_state, with_grads=True)
    names = ["r", "k", "v", "w", "u"]
    leaves = {n: d[n].clone().requires_grad_(grads) for n in names}
    s0 = d.get("init_state")
    if s0 is not None:
        s0 = s0.clone().requires_grad_(grads)
    smap = d.get("state_map") if explicit_map else None
    op = ref6.RWKVKernelOperator(N, T)
    y, s = op(leaves["r"], leaves["k"], leaves["v"], leaves["w"], leaves["u"], with_state=with_state,
              init_state=s0, state_map=smap)
    out = {f"in_{n}": _np(d[n]) for n in names}
    if s0 is not None:
        out["in_init_state"] = _np(s0)
    if smap is not None:
        out["in_state_map"] = smap.numpy()
    out["y"] = _np(y)
    if s is not None:
        out["final_state"] = _np(s)
    if grads:
        loss = (y * d["d_y"]).sum()
        if s is not None:
            loss = loss + (s * d["d_state"]).sum()
            out["d_state"] = _np(d["d_state"])
        loss.backward()
        out["d_y"] = _np(d["d_y"])
        for n in names:
            out[f"grad_{n}"] = _np(leaves[n].grad)
        if s0 is not None:
            out["grad_init_state"] = _np(s0.grad)
    np.savez_compressed(os.path.join(HERE, f"wkv6_{name}.npz"), **out)
    print("wrote", name, y.shape)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of pass-lin/rwkv_ops")
    args = ap.parse_args()
    torch.manual_seed(0)
    torch.set_num_threads(os.cpu_count() or 1)
    ref7 = keras_shim.load_reference_module(
        os.path.join(args.reference, "rwkv_ops/rwkv7_kernel/native_keras_op.py"), "ref_native_rwkv7")
    ref6 = keras_shim.load_reference_module(
        os.path.join(args.reference, "rwkv_ops/rwkv6_kernel/ops_rwkv_kernel.py"), "ref_native_rwkv6")

    # benchmark configuration 0 in full: fp32, B2 T128 H4, per-batch initial state
    rwkv7_case(ref7, "cfg0", 2, 128, 4, seed=1000, state="per_batch")
    # ragged length, no initial state
    rwkv7_case(ref7, "t19_nostate", 1, 19, 2, seed=11)
    # one initial state broadcast over the batch
    rwkv7_case(ref7, "t7_broadcast_state", 2, 7, 2, seed=12, state="broadcast")
    # bf16 inputs (bf16 output, fp32 state)
    rwkv7_case(ref7, "bf16_t64", 2, 64, 2, dtype=torch.bfloat16, seed=13, state="per_batch")
    # single decode step
    rwkv7_case(ref7, "step_t1", 3, 1, 2, seed=14, state="per_batch")

    wkv6_case(ref6, "t33_statemap", 3, 33, 2, seed=21, n_state=2)
    wkv6_case(ref6, "t16_nostate", 2, 16, 2, seed=22, with_state=False)
    wkv6_case(ref6, "t40_cfg4_small", 4, 40, 2, seed=1004, n_state=4)
    wkv6_case(ref6, "t8_defaultmap", 2, 8, 1, seed=23, n_state=2, explicit_map=False)


if __name__ == "__main__":
    main()
