#!/usr/bin/env python3
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `q4k_gemv_4096` is the decode operator: the Q4_K 4096x4096
matrix-vector product (x f32 N(0,1), y f32) over a ring of RING distinct weight
copies (RING x 9.4 MB > the 126 MB L2, so every launch streams its weights from
HBM). One step = one pass over the ring. With N ranks each rank owns its own
ring (independent matvecs, no data-path collective): weak scaling.

Prints ONE JSON line (rank 0). `value` is GB/s of ALGORITHMIC bytes (weights +
x + y per matvec) with everything resident in HBM; `e2e` is the same metric
through the host-pointer C-ABI call jl_matvec (x copied in, y copied out, every
call); `roofline` relates the dominant kernel's achieved GB/s to the measured
HBM peak; `cpu_baseline` is the CPU restatement of the reference's int8 JIT
arithmetic timed on this box's host cores.

`--impl reference` times that CPU path alone (the reference is Go and no Go toolchain
is available to build it) on the same workload and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from jitllm_b200 import synth  # noqa: E402
from jitllm_b200._lib import FLAG_DECODE_CONCURRENT, Q4_K, Q8_0, row_bytes  # noqa: E402

RING = 64
PASSES = 256  # ring passes per step: 16384 matvecs, ~26 ms, so that 20 timed steps run for about half a second
BRANCHES = 8  # parallel branches of the CUDA graph: the ring's matvecs are independent of one another
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu capture of
# this workload's kernel (None until a capture exists for that workload).
NCU_TRAFFIC_BYTES = {"q4k_gemv_4096": 9471232}

WORKLOADS = {
    # name: (type, nrows, k, ntok)
    "q4k_gemv_4096": (Q4_K, 4096, 4096, 1),
}


def algorithmic_bytes(t: int, nrows: int, k: int, ntok: int) -> int:
    return nrows * row_bytes(t, k) + ntok * k * 4 + ntok * nrows * 4


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {}
        for n in ("HwSlowdown", "HwThermalSlowdown", "SwThermalSlowdown", "SwPowerCap", "HwPowerBrakeSlowdown"):
            v = getattr(nv, "nvmlClocksEventReason" + n, None) or getattr(nv, "nvmlClocksThrottleReason" + n, None)
            if v is not None:
                names[v] = n
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, n in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        snake = {"HwSlowdown": "hw_slowdown", "HwThermalSlowdown": "hw_thermal_slowdown",
                 "SwThermalSlowdown": "sw_thermal_slowdown", "SwPowerCap": "sw_power_cap",
                 "HwPowerBrakeSlowdown": "hw_power_brake_slowdown"}
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(snake[r] for r in self.reasons)}


def make_ring(t, nrows, k, ntok, seed, ring):
    rng = synth.rng_for(seed)
    ws = [synth.matrix(rng, t, nrows, k) for _ in range(ring)]
    x = synth.activations(rng, ntok, k)
    return ws, x


def gemv_config(name, world):
    """The `config` object of the headline workload: the same for this library's arm and the reference arm."""
    t, nrows, k, ntok = WORKLOADS[name]
    return {"workload": name, "type": "Q4_K", "nrows": nrows, "k": k, "ntok": ntok, "ring": RING,
            "matvecs_per_step": RING * PASSES,
            "l2": f"inputs larger than L2: ring of {RING} distinct weight copies = {RING * nrows * row_bytes(t, k) / 1e6:.0f} MB",
            "algorithmic_bytes_per_matvec": algorithmic_bytes(t, nrows, k, ntok), "parallelism": f"independent rings x{world}"}


def cpu_ring_rate(ws, x, t, nrows, k, ntok, window, warmup, steps=None, seconds=None):
    """The CPU twin over the ring, all host threads. One CPU step = one pass over the ring of distinct weight
    copies (beyond the host's caches); the rate is bytes over the MEAN step time -- the same statistic in the
    `cpu_baseline` leg and in the reference arm. Runs `steps` steps, or as many as fit `seconds`.
    Returns (GB/s, cores, seconds per step, steps)."""
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    per = algorithmic_bytes(t, nrows, k, ntok)

    def step():
        for w in ws:
            oracle.matmul_int8(t, w, x, nrows, k, ntok, window=window, nthreads=cores)
    for _ in range(warmup):
        step()
    n, t0 = 0, time.perf_counter()
    while (steps is not None and n < steps) or (steps is None and (time.perf_counter() - t0 < seconds or n < 3)):
        step()
        n += 1
    dt = (time.perf_counter() - t0) / n
    return per * len(ws) / dt / 1e9, cores, dt, n


def run_reference(args, name):
    """--impl reference: the reference's CPU path (restated int8 JIT arithmetic) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t, nrows, k, ntok = WORKLOADS[name]
    ws, x = make_ring(t, nrows, k, ntok, 0xB200, RING)   # a CPU step is one pass over the same ring of distinct copies
    val, cores, dt, n = cpu_ring_rate(ws, x, t, nrows, k, ntok, 256 if t == Q4_K else 32, args.warmup, steps=args.steps)
    sample = (f"CPU step = one pass over the ring ({RING} matvecs of {nrows}x{k}, distinct weight copies), {cores} threads, "
              f"mean of {n} steps; the reference is Go and cannot be built here: CPU restatement of its int8-activation "
              "JIT arithmetic (oracle/jl_oracle.c)")
    print(json.dumps({
        "impl": "reference", "metric": "q4k_gemv_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x u4 -> f32",
        "data": "synthetic", "config": gemv_config(name, args.gpus),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def run_ours(args, name):
    import torch
    import torch.distributed as dist
    from jitllm_b200 import Device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import bench_workloads as bw
        bw._pg(local)
    t, nrows, k, ntok = WORKLOADS[name]
    per = algorithmic_bytes(t, nrows, k, ntok)
    ws, x = make_ring(t, nrows, k, ntok, 0xB200 + rank, RING)

    # one context (scratch) per branch; they declare that independent matvecs overlap on the GPU, which
    # selects the decode variant with the most weight bytes in flight. `dev` keeps the defaults: the
    # single dependent chain and the host-pointer end-to-end calls run on it.
    dev = Device(local)
    branch_devs = [Device(local, flags=FLAG_DECODE_CONCURRENT) for _ in range(BRANCHES)]
    for d in branch_devs + [dev]:
        d.Reserve(nrows, k, ntok)
    handles = [dev.Upload(t, w, nrows, k) for w in ws]
    x_dev = torch.from_numpy(x).cuda()
    outs = torch.full((RING, ntok, nrows), float("nan"), device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream()
    sh = stream.cuda_stream

    def ring_pass():
        for i, h in enumerate(handles):
            dev.MatVecDev(outs[i], h, x_dev, ntok, sh)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # One step = PASSES passes over the ring, replayed from a CUDA graph so the launches are
    # back to back on the device (a decode block run is graph-captured in the reference too,
    # jit/gpu/tier/layer.go:6949).
    ring_pass()
    for d in branch_devs:
        d.MatVecDev(outs[0], handles[0], x_dev, ntok, sh)
    torch.cuda.synchronize()

    def capture(branches, devs=None):
        devs = devs or branch_devs
        n0 = sum(d.Stats().launches for d in devs)
        g = torch.cuda.CUDAGraph()
        cap = torch.cuda.Stream()
        side = [torch.cuda.Stream() for _ in range(branches)]
        with torch.cuda.graph(g, stream=cap):
            main = torch.cuda.current_stream()
            for st in side:
                st.wait_stream(main)
            for _ in range(PASSES):
                for i, h in enumerate(handles):
                    b = i % branches
                    devs[b].MatVecDev(outs[i], h, x_dev, ntok, side[b].cuda_stream)
            for st in side:
                main.wait_stream(st)
        return g, sum(d.Stats().launches for d in devs) - n0   # kernels per replay

    graph, kernels_per_replay = capture(BRANCHES)
    chain, _ = capture(1, [dev])   # the same launches as ONE dependent chain (default selection), reported beside the headline
    launches_per_step = RING * PASSES

    def step():
        graph.replay()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        sync_all()
    ms = ev0.elapsed_time(ev1)
    launches = kernels_per_replay * args.steps
    if world > 1:
        tt = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    units = launches_per_step * args.steps
    value = per * units * world / (ms * 1e-3) / 1e9
    kernel_us = ms * 1e3 / units
    for _ in range(3):
        chain.replay()
    torch.cuda.synchronize()
    ev0.record(stream)
    for _ in range(max(2, args.steps // 5)):
        chain.replay()
    ev1.record(stream)
    torch.cuda.synchronize()
    chain_us = ev0.elapsed_time(ev1) * 1e3 / (launches_per_step * max(2, args.steps // 5))
    del graph, chain

    # correctness guard: the timed outputs are real (first ring entry against a second run).
    chk = torch.empty_like(outs[0])
    dev.MatVecDev(chk, handles[0], x_dev, ntok, sh)
    torch.cuda.synchronize()
    assert torch.equal(chk, outs[0]) and bool(torch.isfinite(outs).all()), "timed outputs are not reproducible"

    # end to end: the reference-facing host-pointer call (x in, y out, every call).
    e2e_ring = 8
    out_h = np.empty((ntok, nrows), np.float32)
    for w in ws[:e2e_ring]:
        assert dev.MatVec(out_h, t, w, x, nrows, k), dev.Err()      # uploads (keyed on the host pointer)
    for _ in range(3):
        for w in ws[:e2e_ring]:
            dev.MatVec(out_h, t, w, x, nrows, k)
    n_e2e = max(args.steps, 1) * 4
    # the same public call (jl_matvec, host pointers) issued from a loop inside the library: a Go or C caller pays
    # no interpreter between calls, so neither does this number
    import ctypes as C
    wptrs = (C.c_void_p * e2e_ring)(*[w.ctypes.data for w in ws[:e2e_ring]])
    secs = C.c_double(0.0)
    rc = dev.lib.jl_test_matvec_loop(dev.ctx, out_h.ctypes.data, t, wptrs, ws[0].nbytes, x.ctypes.data, nrows, k, e2e_ring, n_e2e,
                                     C.byref(secs))
    assert rc == 0, dev.Err()
    e2e_s = secs.value
    if world > 1:
        tt = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    e2e_val = per * e2e_ring * n_e2e * world / e2e_s / 1e9

    peak, which = measured_peak()
    line = {
        "metric": "q4k_gemv_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u4 x 2xint8 digits -> s32 (mma.sync u8.s8), f32 fold",
        "data": "synthetic",
        "config": gemv_config(name, world),
        "launch": {"how": f"CUDA graph replay, launches back to back in {BRANCHES} parallel branches (the ring's matvecs are "
                          "independent; programmatic dependent launch inside a branch)",
                   "timed_region_ms": ms,
                   "single_chain_us_per_matvec": chain_us, "single_chain_gbs": per / chain_us / 1e3},
        "roofline": {"bound": "hbm", "achieved": per / (kernel_us * 1e-6) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": per / (kernel_us * 1e-6) / 1e9 / peak, "of": which,
                     "kernel": "gemv_q4k_tma_kernel", "us_per_launch": kernel_us,
                     "us_per_launch_is": "timed region / launches, with 8 launches overlapped on the GPU (not one kernel's duration)",
                     "traffic": NCU_TRAFFIC_BYTES.get(name)},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": ntok * k * 4 * RING * PASSES,
                "d2h_bytes_per_step": ntok * nrows * 4 * RING * PASSES,
                "note": f"jl_matvec host-pointer calls issued from a C loop, {e2e_ring}-copy ring, weights resident, wall clock"},
        "gpu_launches": int(launches),
        "clocks": clk.summary(),
    }
    if rank == 0 and world == 1:
        gbs, cores, dt, n = cpu_ring_rate(ws, x, t, nrows, k, ntok, 256 if t == Q4_K else 32, 2, seconds=10.0)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                "sample": f"CPU step = one pass over the ring ({RING} matvecs of {nrows}x{k}), mean of {n} steps"}
    for h in handles:
        h.free()
    for d in branch_devs + [dev]:
        d.Close()
    del outs, x_dev
    torch.cuda.empty_cache()
    exit_code = 0
    if not args.no_also:
        extra = also_block(args, world, rank, local)
        exit_code = extra.pop("_exit", 0)
        line.update(extra)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        os._exit(exit_code)      # a process group whose collectives were captured in a graph can stall in its destructor
    if exit_code:
        sys.exit(exit_code)


def _brief(line):
    """What the `also` block keeps of a workload's line."""
    if line is None:
        return None
    keep = ("metric", "value", "unit", "ms_per_step", "steps", "scaling", "config", "roofline", "arms", "block_scaled_arm", "e2e",
            "gpu_launches", "clocks")
    return {k: line[k] for k in keep if k in line}


def also_block(args, world, rank, local):
    """The other quantities the metric names, timed in the same run: the prefill GEMM (TFLOP/s against the tensor
    roofline), Q8_0 batch 32, the MXFP4 mixture layer and Llama-3-8B-shaped decode tok/s at batch 1 and 64, each with
    its roofline. Under torchrun they are the SHARDED forms (column-sharded Q8_0, expert-parallel mixture layer,
    tensor-parallel decode: strong scaling), preceded by a parity check of the sharded forms against the unsharded
    ones on the live process group; the run fails when that check is above 2e-3."""
    import bench_workloads as bw
    import copy
    out = {}
    if world > 1:
        par = bw.sharded_parity(local)
        out["sharded_parity"] = par
        if not (par["tp_err"] <= par["bar"] and par["ep_err"] <= par["bar"]):
            # the run fails (exit 3), but the headline line is still printed, with the failed check in it
            par["failed"] = True
            out["_exit"] = 3
            return out
    a = copy.copy(args)
    a.steps, a.warmup = max(args.steps, 20), max(args.warmup, 3)
    also = {}

    def guarded(name, fn):
        """One workload of the block. On one GPU an error in it is recorded in its place and the others still run (the
        headline line must not be lost to a side measurement); under torchrun it propagates, since the other ranks
        would wait in the workload's next collective."""
        try:
            return fn()
        except Exception as e:  # noqa: BLE001
            if world > 1:
                raise
            also[name + "_error"] = f"{type(e).__name__}: {e}"
            return None
    if world == 1:
        also["q4k_gemm_prefill"] = _brief(guarded("q4k_gemm_prefill", lambda: bw.run_gemm(a, emit=False)))
    also["q8_0_batch32"] = _brief(guarded("q8_0_batch32", lambda: bw.run_q8_batch(a, emit=False)))
    also["mxfp4_moe_gptoss"] = _brief(guarded("mxfp4_moe_gptoss", lambda: bw.run_moe(a, emit=False)))
    a.prompt, a.batch = 2048, 1
    lines = guarded("llama8b_q4k_decode", lambda: bw.run_decode(a, emit=False, batches=[1, 64], steps=256))
    for b, l in zip((1, 64), lines or []):
        also[f"llama8b_q4k_decode_b{b}"] = _brief(l)
    out["also"] = also
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="q4k_gemv_4096",
                    choices=sorted(WORKLOADS) + ["q4k_gemm_prefill", "q8_0_batch32", "mxfp4_moe_gptoss", "llama8b_q4k_decode"])
    ap.add_argument("--batch", type=int, default=1, help="llama8b_q4k_decode: sequences decoded together")
    ap.add_argument("--prompt", type=int, default=2048, help="llama8b_q4k_decode: prompt length")
    ap.add_argument("--no-also", action="store_true", help="headline workload only (skip the `also` block)")
    ap.add_argument("--profile", default=None, choices=["gemv", "q8", "gemm", "moe", "block", "attn"],
                    help="run one small fixed case of the named kernel for a profiler to capture (no timing) and exit")
    ap.add_argument("--form", default="auto", choices=["auto", "split", "fused", "wide", "l1", "concurrent"],
                    help="--profile gemv: decode form (concurrent = what the bench's independent branches run)")
    args = ap.parse_args()
    if args.profile:
        import bench_workloads as bw
        bw.profile_case(args)
        return
    if args.workload not in WORKLOADS:
        import bench_workloads as bw
        if args.impl == "reference":
            bw.run_reference(args)
        else:
            {"q4k_gemm_prefill": bw.run_gemm, "q8_0_batch32": bw.run_q8_batch, "mxfp4_moe_gptoss": bw.run_moe, "llama8b_q4k_decode": bw.run_decode}[args.workload](args)
            if int(os.environ.get("WORLD_SIZE", "1")) > 1:
                sys.stdout.flush()
                os._exit(0)
        return
    if args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_ours(args, args.workload)


if __name__ == "__main__":
    main()
