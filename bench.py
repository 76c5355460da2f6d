#!/usr/bin/env python
"""Benchmark of the hot path: RWKV7 generalized delta rule forward + backward, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one forward + backward of ``generalized_delta_rule`` on one batch of synthetic
input (benchmark configuration 1: bf16, B=8, T=4096, H=32, K=V=64, no initial state, upstream
gradients for the output and the final state).  With N > 1 every rank runs the same per-GPU
workload on its own batch (batch x head units are independent: no collective on the data path),
so scaling is weak and ``value`` is the sum over ranks.

Prints ONE JSON line (rank 0).  ``value``: inputs resident in HBM, device-timed with CUDA events,
max over ranks.  ``e2e``: the same metric through the public API with HOST buffers, host->device
and device->host copies of every input and output inside the timed region (``copy_ceiling`` is the
same copies with no compute between them).  ``roofline``: the pass (forward or backward) that holds
the dominant kernel, its algorithmic bytes over the summed CUDA-event time of ALL kernels of that
pass, plus the whole step's fractions of the HBM and tensor peaks.  ``decode`` and ``wkv6``: the other
two measured paths of the metric (T=1 decode of configuration 3, RWKV6 wkv forward + backward of
configuration 4), each with its own roofline.  ``strong_scaling``: configuration 2 with its batch of
16 sequences SHARDED over the ranks (total work fixed).  ``recompute``: the step with the backward
recomputing the forward instead of reading kept tiles.  ``cpu_baseline``: the CPU oracle (a port of
the reference's native operator) timed on this host on a bounded sample.

``--impl reference`` times the reference's own CPU implementation of the path (the oracle port of
``rwkv_ops/rwkv7_kernel/native_keras_op.py``; the reference checkout itself does not travel to the
GPU box) with all host threads, each step a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, T, H, with initial state
    "cfg1": dict(B=8, T=4096, H=32, state=False, desc="rwkv7_fwd_bwd_bf16_B8_T4096_H32_K64"),
    "cfg2": dict(B=16, T=8192, H=64, state=True, desc="rwkv7_fwd_bwd_bf16_B16_T8192_H64_K64_h0_padded"),
}
# algorithmic work per token*head (K = V = 64, bf16 token tensors): forward reads 6 and writes 1
# vector of 128 B, backward reads 7 and writes 6
BYTES_PER_TOKEN_HEAD = 2560
FLOP_PER_TOKEN_HEAD = 434176
# DRAM traffic (dram__bytes_read + dram__bytes_write, ncu) per chunk-head (64 tokens of one head) of each
# chunked kernel, captured on a small case (B=2, T=4096, H=16); traffic grows in proportion to the number of
# chunk-heads, so a full launch is this figure times B*H*ceil(T/64).
TRAFFIC_PER_CHUNK_HEAD = {"r7c_intra_fwd_kernel": 112.1e3, "r7c_scan_fwd_kernel": 85.2e3,
                          "r7c_bwd_pre_kernel": 35.5e3, "r7c_bwd_scan_kernel": 47.9e3,
                          "r7c_bwd_final_kernel": 149.8e3}
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum per chunk-head on B=2 T=4096 H=16 "
                  "(a full-size launch is too large to capture), scaled by the chunk-heads of this launch")


def cores_near_gpu(dev):
    """The CPU cores NVML reports as local to CUDA device `dev` (its NUMA node), restricted to the cores this
    process may run on; None when that cannot be found out.  Reads only."""
    try:
        import pynvml
        pynvml.nvmlInit()
        p = torch.cuda.get_device_properties(dev)
        bus = f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        return cpus if len(cpus) >= 2 else None
    except Exception:      # noqa: BLE001  (no NVML, no such call, a container that hides the topology)
        return None


CPU_SAMPLE_T = 256     # tokens per sequence of the cpu_baseline sample
REF_STEP_T = 128       # tokens per sequence of one --impl reference step


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._th = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv is not None:
            self._th = threading.Thread(target=self._run, daemon=True)
            self._th.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._th is not None:
            self._th.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_reference_step(B, T, H, with_state, seed, state=None, return_state=False):
    """One forward + backward of the CPU oracle (port of the reference's native operator) over a block
    of T tokens per sequence; ``state`` chains blocks of one sequence (the recurrence is Markov)."""
    from oracle import generalized_delta_rule as oracle_gdr
    from rwkv_ops_b200.workloads import rwkv7_inputs
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=seed, with_state=with_state, with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    h0 = state if state is not None else d.get("initial_state")
    t0 = time.perf_counter()
    o, s = oracle_gdr(*[g[n] for n in "rwkvab"], initial_state=h0)
    ((o.float() * d["d_out"].float()).sum() + (s * d["d_state"]).sum()).backward()
    sec = time.perf_counter() - t0
    return (sec, s.detach()) if return_state else sec


def cpu_baseline_sample(B, T, H, with_state, budget_s=12.0):
    """The oracle over consecutive blocks of CPU_SAMPLE_T tokens of every sequence (state chained from
    block to block, forward + backward per block) until ``budget_s`` seconds of work or the whole
    sequence length.  Returns (tokens per second, description)."""
    cpu_reference_step(B, 16, H, with_state, 5)   # warm the allocator and thread pool
    total, blocks, state = 0.0, 0, None
    while blocks * CPU_SAMPLE_T < T and total < budget_s:
        sec, state = cpu_reference_step(B, min(CPU_SAMPLE_T, T - blocks * CPU_SAMPLE_T), H, with_state,
                                        6 + blocks, state=state, return_state=True)
        total += sec
        blocks += 1
    ntok = min(T, blocks * CPU_SAMPLE_T)
    return B * ntok / total, (f"B={B} H={H} first {ntok} of {T} tokens per sequence in {blocks} block(s) of "
                              f"{CPU_SAMPLE_T} with the state chained, fwd+bwd per block, float32 CPU, {total:.1f} s")


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B, H, T = wl["B"], wl["H"], REF_STEP_T
    for i in range(args.warmup):
        cpu_reference_step(B, T, H, wl["state"], 10 + i)
    total = 0.0
    for i in range(args.steps):
        total += cpu_reference_step(B, T, H, wl["state"], 100 + i)
    ms = 1e3 * total / args.steps
    val = B * T / (ms / 1e3)
    sample = f"B={B} H={H} first {T} of {wl['T']} tokens per sequence, fwd+bwd, float32 CPU"
    line = {
        "impl": "reference", "metric": "rwkv7_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["desc"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _timed(fn, steps, warmup, barrier, max_over_ranks):
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return max_over_ranks(e0.elapsed_time(e1)) / steps


def sub_decode(dev, world, max_over_ranks, barrier, pk):
    """Configuration 3: T=1 decode, B=256, H=64, bf16 tokens, float32 state fed back over 1024 consecutive
    steps (ping-pong state buffers of 268 MB each, larger than L2; 8 rotating sets of token vectors)."""
    from rwkv_ops_b200 import _lib
    from rwkv_ops_b200.workloads import rwkv7_inputs
    B, H, STEPS = 256, 64, 1024
    lib = _lib.load()
    ds = [rwkv7_inputs(B, 1, H, dtype=torch.bfloat16, seed=1003 + i, device=dev) for i in range(8)]
    bufs = [0.1 * torch.randn(B, H, 64, 64, device=dev), torch.empty(B, H, 64, 64, device=dev)]
    o = torch.empty(B, H, 64, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    i = [0]

    def fn():
        d = ds[i[0] & 7]
        rc = lib.rwkvb200_rwkv7_step(*[d[n].data_ptr() for n in "rwkvab"], bufs[i[0] & 1].data_ptr(), B,
                                     bufs[(i[0] + 1) & 1].data_ptr(), o.data_ptr(), B, H, 64, _lib.BF16, st)
        assert rc == 0
        i[0] += 1

    ms = _timed(fn, STEPS, 8, barrier, max_over_ranks)
    nbytes = B * H * (2 * 64 * 64 * 4 + 7 * 64 * 2)
    gbs = nbytes / (ms / 1e3) / 1e9
    return {"workload": "rwkv7_decode_T1_bf16_B256_H64_f32_state", "steps": STEPS, "us_per_step": 1e3 * ms,
            "value": gbs, "unit": "GB/s per GPU", "tokens_per_s": world * B / (ms / 1e3),
            "roofline": {"bound": "hbm", "algorithmic_bytes": nbytes, "achieved": gbs, "peak": pk["hbm_gbs"],
                         "frac": gbs / pk["hbm_gbs"], "kernel": "rwkv7_step_kernel"}}


def sub_wkv6(dev, world, max_over_ranks, barrier, pk):
    """Configuration 4: RWKV6 wkv forward + backward, fp32, B=16, T=4096, 32 heads, 4 initial states
    selected through state_map; algorithmic bytes 14 fp32 vectors of 256 B per token*head."""
    import rwkv_ops_b200 as ro
    from rwkv_ops_b200 import _lib
    from rwkv_ops_b200.workloads import wkv6_inputs
    B, T, H = 16, 4096, 32
    d = wkv6_inputs(B, T, H, seed=1004, device=dev, n_state=4, with_grads=True)
    g = {n: d[n].requires_grad_(True) for n in "rkvwu"}
    s0 = d["init_state"].requires_grad_(True)
    op = ro.RWKV6_OP(64, T)

    def fn():
        y, s = op(g["r"], g["k"], g["v"], g["w"], g["u"], with_state=True, init_state=s0, state_map=d["state_map"])
        torch.autograd.backward([y, s], [d["d_y"], d["d_state"]])
        for t in list(g.values()) + [s0]:
            t.grad = None

    for _ in range(3):
        fn()
    _lib.profile(True)
    ms = _timed(fn, 5, 0, barrier, max_over_ranks)
    prof = _lib.profile_results()
    _lib.profile(False)
    nbytes = B * T * H * 3584
    gbs = nbytes / (ms / 1e3) / 1e9
    return {"workload": "wkv6_fwd_bwd_f32_B16_T4096_C2048_4states", "ms_per_step": ms,
            "value": world * B * T / (ms / 1e3), "unit": "tokens/s",
            "kernels": {k_: v[0] / 5 for k_, v in prof.items()},
            "roofline": {"bound": "hbm", "algorithmic_bytes": nbytes, "achieved": gbs, "peak": pk["hbm_gbs"],
                         "frac": gbs / pk["hbm_gbs"], "kernel": "wkv6c_bwd_kernel"}}


def sub_cfg2_sharded(dev, world, rank, max_over_ranks, barrier):
    """Configuration 2 (bf16, B=16, T=8192, H=64, per-sequence initial state, trailing 0..512 tokens padded
    through w): the 16 sequences are sharded over the ranks (B/N per rank, no collective), so the total work
    is the same at every N.  value = tokens of all 16 sequences / max over ranks of the step time."""
    import rwkv_ops_b200 as ro
    from rwkv_ops_b200.workloads import rwkv7_inputs, rwkv7_pad_lengths, apply_w_padding
    Bg, T, H = 16, 8192, 64
    if Bg % world:
        return {"skipped": f"{Bg} sequences do not divide over {world} ranks"}
    Bl = Bg // world
    d = rwkv7_inputs(Bl, T, H, dtype=torch.bfloat16, seed=1002 + 17 * rank, device=dev, with_state=True,
                     with_grads=True)
    lengths = rwkv7_pad_lengths(Bg, T, seed=1002)[rank * Bl:(rank + 1) * Bl]
    d["w"] = apply_w_padding(d["w"], lengths)
    leaves = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].requires_grad_(True)

    def fn():
        o, s = ro.generalized_delta_rule(*[leaves[n] for n in "rwkvab"], initial_state=h0)
        torch.autograd.backward([o, s], [d["d_out"], d["d_state"]])
        for n in "rwkvab":
            leaves[n].grad = None
        h0.grad = None

    ms = _timed(fn, 5, 3, barrier, max_over_ranks)
    out = {"workload": "rwkv7_fwd_bwd_bf16_B16_T8192_H64_K64_h0_padded", "scaling": "strong",
           "sharding": f"{Bl} of 16 sequences per rank, {world} rank(s), no collective",
           "ms_per_step": ms, "value": Bg * T / (ms / 1e3), "unit": "tokens/s",
           "units_per_gpu": Bl * H}
    del d, leaves, h0
    torch.cuda.empty_cache()
    return out


def sub_cfg2_sequence_parallel(dev, world, rank, max_over_ranks, barrier):
    """Configuration 2 with every sequence's 8192 tokens split over the ranks (rank g holds tokens
    [g*T/N, (g+1)*T/N) of all 16 sequences); the boundary states and their gradients travel between
    neighbours by NCCL point-to-point.  value = tokens of all 16 sequences / max over ranks of the step."""
    import torch.distributed as dist
    from rwkv_ops_b200.sequence_parallel import generalized_delta_rule_sp
    from rwkv_ops_b200.workloads import rwkv7_inputs
    B, T, H = 16, 8192, 64
    if T % (64 * world):
        return {"skipped": f"{T} tokens do not split into whole chunks over {world} ranks"}
    Tl = T // world
    d = rwkv7_inputs(B, Tl, H, dtype=torch.bfloat16, seed=1002 + 31 * rank, device=dev, with_state=True,
                     with_grads=True)
    leaves = {n: d[n].requires_grad_(True) for n in "rwkvab"}
    h0 = d["initial_state"].requires_grad_(True) if rank == 0 else None
    d_state = d["d_state"] if rank == world - 1 else None

    def fn():
        o, s = generalized_delta_rule_sp(*[leaves[n] for n in "rwkvab"], initial_state=h0)
        if d_state is not None:
            torch.autograd.backward([o, s], [d["d_out"], d_state])
        else:
            torch.autograd.backward([o], [d["d_out"]])
        for n in "rwkvab":
            leaves[n].grad = None
        if h0 is not None:
            h0.grad = None

    ms = _timed(fn, 5, 3, barrier, max_over_ranks)
    out = {"workload": "rwkv7_fwd_bwd_bf16_B16_T8192_H64_K64_h0_sequence_parallel", "scaling": "strong",
           "sharding": f"{Tl} of 8192 tokens of every sequence per rank, {world} rank(s), boundary states by "
                       "NCCL send/recv into the receiver's own memory",
           "ms_per_step": ms, "value": B * T / (ms / 1e3), "unit": "tokens/s"}
    del d, leaves
    torch.cuda.empty_cache()
    return out


def run_ours(args, wl):
    import torch.distributed as dist
    import rwkv_ops_b200 as ro
    from rwkv_ops_b200 import _lib
    from rwkv_ops_b200.workloads import rwkv7_inputs, rwkv7_pad_lengths, apply_w_padding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # the NCCL backend announces its version on stdout when its first communicator is made; stdout is for the
        # one JSON line, so that goes to stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    _lib.load()

    B, T, H = wl["B"], wl["T"], wl["H"]
    d = rwkv7_inputs(B, T, H, dtype=torch.bfloat16, seed=1001 + rank, device=dev, with_state=wl["state"],
                     with_grads=True)
    if wl["state"]:   # configuration 2 pads the trailing 0..512 tokens of every sequence through w
        d["w"] = apply_w_padding(d["w"], rwkv7_pad_lengths(B, T, seed=1002 + rank))
    names = "rwkvab"
    leaves = {n: d[n].requires_grad_(True) for n in names}
    h0 = d.get("initial_state")
    if h0 is not None:
        h0.requires_grad_(True)
    d_out, d_state = d["d_out"], d["d_state"]

    def step():
        o, s = ro.generalized_delta_rule(*[leaves[n] for n in names], initial_state=h0)
        torch.autograd.backward([o, s], [d_out, d_state])
        for n in names:
            leaves[n].grad = None
        if h0 is not None:
            h0.grad = None
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # ---- device-resident throughput
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.profile(True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    prof = _lib.profile_results()
    _lib.profile(False)
    ms_step = ms_total / args.steps
    value = world * B * T / (ms_step / 1e3)
    launches = sum(n for _, n in prof.values())

    # ---- roofline.  The dominant kernel (by summed event time inside the timed region) names the pass;
    # the pass's algorithmic bytes (forward: 6 vectors of 128 B read + 1 written per token*head = 896 B;
    # backward: 7 read + 6 written = 1664 B) are divided by the summed time of ALL kernels of that pass.
    pk = peaks()
    roof = None
    units = B * T * H
    if prof:
        per_step = {k_: v[0] / args.steps for k_, v in prof.items()}
        top = max(per_step, key=per_step.get)
        is_bwd = "bwd" in top
        members = [k_ for k_ in per_step if ("bwd" in k_) == is_bwd]
        pass_ms = sum(per_step[k_] for k_ in members)
        bytes_per_unit = 1664 if is_bwd else 896
        achieved = units * bytes_per_unit / (pass_ms / 1e3) / 1e9
        n_ch = B * H * ((T + 63) // 64)
        traffic = sum(TRAFFIC_PER_CHUNK_HEAD.get(k_, 0.0) for k_ in members) * n_ch
        step_gbs = units * BYTES_PER_TOKEN_HEAD / (ms_step / 1e3) / 1e9
        step_tf = units * FLOP_PER_TOKEN_HEAD / (ms_step / 1e3) / 1e12
        roof = {"kernel": top, "pass": "backward" if is_bwd else "forward", "pass_kernels": sorted(members),
                "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "traffic": traffic or None,
                "traffic_source": TRAFFIC_SOURCE,
                "algorithmic_bytes": units * bytes_per_unit, "peak_source": pk["source"],
                "pass_ms": pass_ms, "launch_ms": per_step[top],
                "step": {"algorithmic_bytes": units * BYTES_PER_TOKEN_HEAD, "hbm_gbs": step_gbs,
                         "hbm_frac": step_gbs / pk["hbm_gbs"], "flop": units * FLOP_PER_TOKEN_HEAD,
                         "tensor_tflops": step_tf, "tensor_frac": step_tf / pk["bf16_tflops"]},
                "kernels": {k_: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                            for k_, v in prof.items()}}

    # ---- the same step with the backward recomputing the forward (nothing kept between the passes)
    kept_bytes = _lib.load().rwkvb200_rwkv7_fwd_workspace_bytes(B, T, H, 64, _lib.BF16, _lib.ALGO_KEEP)
    os.environ["RWKV_OPS_B200_KEEP_LIMIT_MB"] = "0"
    for _ in range(2):
        step()
    barrier()
    ev0.record()
    for _ in range(max(3, args.steps // 2)):
        step()
    ev1.record()
    barrier()
    recompute_ms = max_over_ranks(ev0.elapsed_time(ev1)) / max(3, args.steps // 2)
    del os.environ["RWKV_OPS_B200_KEEP_LIMIT_MB"]

    extra = {}
    if not args.only_main:
        subs = [("decode", lambda: sub_decode(dev, world, max_over_ranks, barrier, pk)),
                ("wkv6", lambda: sub_wkv6(dev, world, max_over_ranks, barrier, pk)),
                ("strong_scaling", lambda: sub_cfg2_sharded(dev, world, rank, max_over_ranks, barrier))]
        if world > 1:
            subs.append(("sequence_parallel",
                         lambda: sub_cfg2_sequence_parallel(dev, world, rank, max_over_ranks, barrier)))
        for name, fn in subs:
            try:      # a sub-record that cannot run (e.g. out of memory) must not cost the main line
                extra[name] = fn()
            except Exception as exc:      # noqa: BLE001
                extra[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                torch.cuda.empty_cache()

    # ---- end to end: host buffers in, host buffers out, through the public API.
    # Every step copies all of its inputs from pinned host memory and all of its results back to
    # pinned host memory.  Steps are independent, so they are software-pipelined over three streams:
    # the upload of step i+1 and the download of step i-1 overlap the compute of step i (PCIe is
    # full duplex); two sets of device and host buffers alternate.
    # The pinned buffers are allocated (and first touched) while the process is bound to the cores of the GPU's
    # own NUMA node, so that with several ranks on a multi-socket host no rank copies across sockets.
    near = cores_near_gpu(dev)
    before = os.sched_getaffinity(0)
    if near:
        os.sched_setaffinity(0, near)
    host_in = {n: d[n].detach().to("cpu").pin_memory() for n in names}
    host_in["d_out"] = d_out.to("cpu").pin_memory()
    host_in["d_state"] = d_state.to("cpu").pin_memory()
    if h0 is not None:
        host_in["h0"] = h0.detach().to("cpu").pin_memory()
    out_names = list(names) + ["o", "ht"] + (["dh0"] if h0 is not None else [])

    def host_out_set():
        ho = {n: torch.empty_like(host_in[n]).pin_memory() for n in names}
        ho["o"] = torch.empty_like(host_in["r"]).pin_memory()
        ho["ht"] = torch.empty(B, H, 64, 64).pin_memory()
        if h0 is not None:
            ho["dh0"] = torch.empty_like(host_in["h0"]).pin_memory()
        return ho

    host_out = [host_out_set(), host_out_set()]
    if near:
        os.sched_setaffinity(0, before)
    dev_in = [{n: torch.empty_like(t, device=dev) for n, t in host_in.items()} for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out[0].values())
    s_up, s_run, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]
    results = [None, None]

    def e2e_run(nsteps):
        for i in range(nsteps):
            sl = i & 1
            with torch.cuda.stream(s_up):
                s_up.wait_event(ev_run[sl])          # the compute that last read this input set is done
                for n, t in host_in.items():
                    dev_in[sl][n].copy_(t, non_blocking=True)
                ev_up[sl].record(s_up)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_up[sl])
                s_run.wait_event(ev_down[sl])        # the download that last read this result set is done
                dv = dev_in[sl]
                lv = {n: dv[n].detach().requires_grad_(True) for n in names}
                s0 = dv.get("h0")
                if s0 is not None:
                    s0 = s0.detach().requires_grad_(True)
                o, s = ro.generalized_delta_rule(*[lv[n] for n in names], initial_state=s0)
                torch.autograd.backward([o, s], [dv["d_out"], dv["d_state"]])
                res = {n: lv[n].grad for n in names}
                res["o"], res["ht"] = o.detach(), s.detach()
                if s0 is not None:
                    res["dh0"] = s0.grad
                results[sl] = res
                ev_run[sl].record(s_run)
            with torch.cuda.stream(s_down):
                s_down.wait_event(ev_run[sl])
                for n in out_names:
                    host_out[sl][n].copy_(results[sl][n], non_blocking=True)
                    results[sl][n].record_stream(s_down)
                ev_down[sl].record(s_down)
        for st_ in (s_up, s_run, s_down):
            st_.synchronize()                        # every result is in host memory

    # enough steps that the fill and drain of the three-stage pipeline (one upload before the first compute,
    # one download after the last) weigh a few per cent, not ten
    e2e_steps = max(24, min(args.steps, 50))
    e2e_run(3)
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    e2e_run(e2e_steps)
    ev1.record()
    barrier()
    e2e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), 1e3 * (time.perf_counter() - t0))) / e2e_steps
    e2e_val = world * B * T / (e2e_ms / 1e3)

    # copy-only ceiling of the same host path: the same pinned buffers up and down on the two copy
    # streams, no compute between them
    dev_out = {n: torch.empty_like(t, device=dev) for n, t in host_out[0].items()}

    def copy_only(nsteps):
        for i in range(nsteps):
            sl = i & 1
            with torch.cuda.stream(s_up):
                for n, t in host_in.items():
                    dev_in[sl][n].copy_(t, non_blocking=True)
            with torch.cuda.stream(s_down):
                for n in out_names:
                    host_out[sl][n].copy_(dev_out[n], non_blocking=True)
        s_up.synchronize()
        s_down.synchronize()

    copy_only(2)
    barrier()
    t0 = time.perf_counter()
    copy_only(e2e_steps)
    barrier()
    copy_ms = max_over_ranks(1e3 * (time.perf_counter() - t0)) / e2e_steps

    if rank == 0:
        line = {
            "metric": "rwkv7_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["desc"], "per_gpu_batch": B, "seq_len": T, "heads": H,
                       "sharding": f"batch x head units replicated per GPU, {world} rank(s), no collective",
                       "l2": f"inputs ({7 * B * T * H * 64 * 2 / 1e9:.2f} GB per step) exceed the 126 MB L2",
                       "algo": os.environ.get("RWKV_OPS_B200_RWKV7_ALGO", "auto")},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "pipeline": "upload / compute / download of consecutive steps overlap on three streams",
                    "host_buffers": (f"pinned while bound to the {len(near)} cores NVML reports as local to the GPU"
                                     if near else "pinned where the process ran (no NVML core affinity found)"),
                    "copy_ceiling": {"ms_per_step": copy_ms, "value": world * B * T / (copy_ms / 1e3),
                                     "frac_of_ceiling": copy_ms / e2e_ms,
                                     "what": "the same pinned host buffers copied up and down, no compute"}},
            "gpu_launches": launches,
            "roofline": roof,
            "recompute": {"ms_per_step": recompute_ms, "value": world * B * T / (recompute_ms / 1e3),
                          "kept_bytes_per_step": int(kept_bytes),
                          "what": "backward recomputes the forward from the inputs (nothing saved but inputs)"},
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            val, sample = cpu_baseline_sample(B, T, H, wl["state"])
            line["cpu_baseline"] = {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-main", action="store_true", help="skip the decode / wkv6 / strong-scaling sub-records")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
