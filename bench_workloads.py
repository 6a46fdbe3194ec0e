"""The other measured workloads of the quantized-matmul path, behind `bench.py --workload ...`:

  q4k_gemm_prefill     Q4_K x bf16 GEMM, 512 tokens, 14336x4096 and 4096x14336       (TFLOP/s, tensor roofline)
  q8_0_batch32         Q8_0 batched decode, 32 tokens, 4096->4096 / 1024 / 14336          (weight GB/s; column-sharded under torchrun)
  mxfp4_moe_gptoss     MXFP4 mixture layer 32 experts / top-4 / 2880 / 256 tokens     (layers/s + weight GB/s, HBM roofline)
  llama8b_q4k_decode   Llama-3-8B-shaped Q4_K decoder, 2048-token prompt, greedy decode (tok/s; tensor-parallel under torchrun)

Each prints one JSON line with the same keys as the headline workload. Inputs are seeded synthetic tensors
of the stated shapes; every timed region is a CUDA-graph replay timed with CUDA events on the launching stream,
with working sets larger than L2.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import time

import numpy as np


def _env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return world, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def _pg(local):
    """The process group of a torchrun launch, created once per process (NCCL, one rank per GPU)."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return dist


def _emit(line, emit):
    if emit and line is not None:
        print(json.dumps(line), flush=True)
    return line


def _peaks():
    import bench
    p = os.path.join(bench.ROOT, "MEASURED_PEAKS.json")
    d = json.load(open(p)) if os.path.exists(p) else {}
    return (float(d.get("hbm_gbs", bench.FALLBACK_HBM_GBS)), float(d.get("bf16_tflops", 1590.0)),
            float(d.get("bf16_tflops_sustained", 1400.0)), "measured" if d else "fallback")


def _timed_replays(torch, graph, steps, warmup, local):
    import bench
    for _ in range(max(warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with bench.ClockSampler(local) as clk:
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1), clk.summary()


# ------------------------------------------------------------------ prefill GEMM
GEMM_SHAPES = [(14336, 4096), (4096, 14336)]
GEMM_NTOK, GEMM_COPIES = 512, 6          # 6 distinct weight copies per shape: 198 MB > L2


def run_gemm(args, emit=True):
    import torch
    from jitllm_b200 import Device, synth
    from jitllm_b200._lib import Q4_K
    world, rank, local = _env()
    if rank != 0:
        return None     # single-GPU workload: replicas would only repeat it
    torch.cuda.set_device(local)
    dev = Device(local)
    rng = synth.rng_for(0xB201)
    sh = torch.cuda.current_stream().cuda_stream
    sets, flops = [], 0.0
    for nrows, k in GEMM_SHAPES:
        dev.Reserve(nrows, k, GEMM_NTOK)
        hs = [dev.Upload(Q4_K, synth.q4k_matrix(rng, nrows, k), nrows, k) for _ in range(GEMM_COPIES)]
        x = torch.randn(GEMM_NTOK, k, device="cuda").to(torch.bfloat16)
        out = torch.empty(GEMM_NTOK, nrows, device="cuda", dtype=torch.bfloat16)
        for h in hs:
            dev.MatMulDev(out, h, x, GEMM_NTOK, sh)
        sets.append((hs, x, out))
        flops += 2.0 * GEMM_NTOK * nrows * k * GEMM_COPIES
    torch.cuda.synchronize()
    n0 = dev.Stats().launches
    g, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=cap):
        c = torch.cuda.current_stream().cuda_stream
        for hs, x, out in sets:
            for h in hs:
                dev.MatMulDev(out, h, x, GEMM_NTOK, c)
    per_replay = dev.Stats().launches - n0
    ms, clocks = _timed_replays(torch, g, args.steps, args.warmup, local)
    tf = flops * args.steps / (ms * 1e-3) / 1e12
    # end to end: host bf16 activations in, host bf16 outputs back, weights resident (keyed on the host pointer)
    nrows, k = GEMM_SHAPES[0]
    w_host = synth.q4k_matrix(rng, nrows, k)
    x_host = synth.to_bf16_bits(synth.activations(rng, GEMM_NTOK, k))
    out_host = np.empty((GEMM_NTOK, nrows), np.uint16)
    assert dev.MatMulRaw(out_host, 2, Q4_K, w_host, x_host, 2, nrows, k, GEMM_NTOK), dev.Err()
    n_e2e = 20
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        dev.MatMulRaw(out_host, 2, Q4_K, w_host, x_host, 2, nrows, k, GEMM_NTOK)
    e2e_tf = 2.0 * GEMM_NTOK * nrows * k * n_e2e / (time.perf_counter() - t0) / 1e12
    hbm, burst, sustained, which = _peaks()
    ngemm = len(GEMM_SHAPES) * GEMM_COPIES
    line = ({
        "metric": "q4k_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "Q4_K -> f16 weights x bf16->f16 activations, f32 accumulate (tcgen05 kind::f16), bf16 out",
        "data": "synthetic",
        "config": {"workload": "q4k_gemm_prefill", "ntok": GEMM_NTOK, "shapes": GEMM_SHAPES, "copies_per_shape": GEMM_COPIES,
                   "l2": "6 distinct weight copies per shape (198 MB) cycle through: larger than L2",
                   "us_per_gemm": ms * 1e3 / args.steps / ngemm},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst, "of": which,
                     "frac_of_sustained": tf / sustained, "kernel": "gemm_q4k_tc5_kernel", "traffic": None},
        "e2e": {"value": e2e_tf, "unit": "TFLOP/s", "h2d_bytes_per_step": GEMM_NTOK * k * 2,
                "d2h_bytes_per_step": GEMM_NTOK * nrows * 2, "note": "jl_matmul host-pointer call, 14336x4096, wall clock"},
        "gpu_launches": int(per_replay * args.steps), "clocks": clocks})
    for hs, _, _ in sets:
        for h in hs:
            h.free()
    dev.Close()
    return _emit(line, emit)


# ------------------------------------------------------------------ Q8_0 batched decode
Q8_SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096)]
Q8_NTOK = 32


def run_q8_batch(args, emit=True):
    """Q8_0 batch-32 decode matmuls (f32 activations), the three shapes back to back over rings of distinct
    weight copies. Under torchrun the rows are column-sharded over the ranks (strong scaling, no collective)."""
    import torch
    from jitllm_b200 import Device, synth
    from jitllm_b200._lib import Q8_0
    world, rank, local = _env()
    torch.cuda.set_device(local)
    if world > 1:
        dist = _pg(local)
    dev = Device(local)
    rng = synth.rng_for(0xB202 + rank)
    sh = torch.cuda.current_stream().cuda_stream
    sets, wbytes, flops = [], 0, 0.0
    for nrows_full, k in Q8_SHAPES:
        nrows = nrows_full // world
        copies = max(2, int(200e6 / (nrows * k * 34 / 32)) + 1)           # each ring beyond L2
        dev.Reserve(nrows, k, Q8_NTOK)
        hs = [dev.Upload(Q8_0, synth.q8_0_matrix(rng, nrows, k), nrows, k) for _ in range(copies)]
        x = torch.randn(Q8_NTOK, k, device="cuda")
        out = torch.empty(Q8_NTOK, nrows, device="cuda")
        for h in hs:
            dev.MatMulDev(out, h, x, Q8_NTOK, sh)
        sets.append((hs, x, out))
        wbytes += copies * (nrows * k * 34 // 32 + Q8_NTOK * (k + nrows) * 4)
        flops += 2.0 * Q8_NTOK * nrows * k * copies
    torch.cuda.synchronize()
    n0 = dev.Stats().launches
    g, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=cap):
        c = torch.cuda.current_stream().cuda_stream
        for hs, x, out in sets:
            for h in hs:
                dev.MatMulDev(out, h, x, Q8_NTOK, c)
    per_replay = dev.Stats().launches - n0
    if world > 1:
        dist.barrier()
    ms, clocks = _timed_replays(torch, g, args.steps, args.warmup, local)
    if world > 1:
        tt = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt)
    gbs = wbytes * args.steps / (ms * 1e-3) / 1e9          # per rank
    # end to end on the 4096x4096 shard: host activations in, host outputs back
    nrows, k = Q8_SHAPES[0][0] // world, Q8_SHAPES[0][1]
    w_host, x_host = synth.q8_0_matrix(rng, nrows, k), synth.activations(rng, Q8_NTOK, k)
    out_host = np.empty((Q8_NTOK, nrows), np.float32)
    assert dev.MatMul(out_host, Q8_0, w_host, x_host, nrows, k, Q8_NTOK), dev.Err()
    t0 = time.perf_counter()
    for _ in range(50):
        dev.MatMul(out_host, Q8_0, w_host, x_host, nrows, k, Q8_NTOK)
    e2e = 50 * (nrows * k * 34 // 32 + Q8_NTOK * (k + nrows) * 4) / (time.perf_counter() - t0) / 1e9
    hbm, burst, sustained, which = _peaks()
    line = None
    if rank == 0:
        line = ({
            "metric": "q8_0_batch32_gbs", "value": gbs * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "s8 codes x two int8 digits per activation (mma.sync m16n8k32), d and 1/s folded in f32",
            "data": "synthetic",
            "config": {"workload": "q8_0_batch32", "ntok": Q8_NTOK, "shapes": Q8_SHAPES, "parallelism": f"column-parallel x{world}",
                       "l2": "a ring of distinct weight copies per shape, each ring > 200 MB: larger than L2",
                       "tflops": flops * args.steps / (ms * 1e-3) / 1e12 * world},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "of": which,
                         "kernel": "q8_xprep_kernel + gemv_q8_batch_kernel (k-slices summed inside a cluster)", "traffic": None},
            "e2e": {"value": e2e * world, "unit": "GB/s", "h2d_bytes_per_step": Q8_NTOK * k * 4, "d2h_bytes_per_step": Q8_NTOK * nrows * 4,
                    "note": "jl_matmul host-pointer call on the 4096x4096 shard, wall clock"},
            "gpu_launches": int(per_replay * args.steps), "clocks": clocks})
    for hs, _, _ in sets:
        for h in hs:
            h.free()
    dev.Close()
    if world > 1:
        dist.barrier()
    return _emit(line, emit)


# ------------------------------------------------------------------ mixture layer
MOE = dict(E=32, topk=4, hidden=2880, ffn=2880, ntok=256, layers=2)   # 2 distinct layers: 846 MB of experts > L2


def run_moe_ep(args, emit=True):
    """The same layer expert-parallel under torchrun: 32 / world experts per rank, the 256 tokens data-parallel,
    NCCL all-to-all dispatch and return, combine in ascending expert id on the token's home rank."""
    import torch
    import torch.distributed as dist
    from jitllm_b200 import Device, parallel, synth
    from jitllm_b200._lib import MXFP4, MoeDesc
    world, rank, local = _env()
    torch.cuda.set_device(local)
    _pg(local)
    E, topk, hidden, ffn, ntok_all = MOE["E"], MOE["topk"], MOE["hidden"], MOE["ffn"], MOE["ntok"]
    epr, ntok = E // world, ntok_all // world
    rng = synth.rng_for(0xB203 + rank)
    dev = Device(local)
    stream = torch.cuda.current_stream().cuda_stream
    hs = [dev.Upload(MXFP4, synth.mxfp4_matrix(rng, epr * r, kk), r, kk, epr) for r, kk in ((ffn, hidden), (ffn, hidden), (hidden, ffn))]
    dev.MoeReserve(ntok_all * topk, max(E, epr), topk, hidden, ffn)
    d_route = MoeDesc(struct_size=C.sizeof(MoeDesc), type=MXFP4, n_expert=E, top_k=topk, hidden=hidden, ffn=ffn, act=0, norm=1, scale=1.0)
    from jitllm_b200._lib import MOE_ARM_BLOCK_SCALED_X3
    d_local = MoeDesc(struct_size=C.sizeof(MoeDesc), type=MXFP4, n_expert=epr, top_k=1, hidden=hidden, ffn=ffn, act=0, norm=1,
                      scale=1.0, gate=hs[0].handle, up=hs[1].handle, down=hs[2].handle, arm=MOE_ARM_BLOCK_SCALED_X3)

    def route(lg):
        sel = torch.empty(lg.shape[0], topk, dtype=torch.int32, device="cuda")
        wt = torch.empty(lg.shape[0], topk, dtype=torch.float32, device="cuda")
        dev.MoeRouteDev(lg, lg.shape[0], d_route, sel, wt, torch.cuda.current_stream().cuda_stream)
        return sel, wt

    def experts(rows, ids):
        y = torch.empty(rows.shape[0], hidden, dtype=torch.float32, device="cuda")
        dev.MoeExpertsDev(y, rows.contiguous(), ids.contiguous(), rows.shape[0], d_local, torch.cuda.current_stream().cuda_stream)
        return y
    moe = parallel.ExpertParallelMoE(route, experts, E, topk, hidden)
    g = torch.Generator(device="cuda").manual_seed(11 + rank)
    h = torch.randn(ntok, hidden, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(ntok, E, device="cuda", generator=g)
    out = torch.zeros(ntok, hidden, device="cuda")
    n0 = dev.Stats().launches
    for _ in range(max(args.warmup, 3)):
        moe.forward(out, h, logits)
    per_step = (dev.Stats().launches - n0) // max(args.warmup, 3)
    dist.barrier()
    torch.cuda.synchronize()
    # the layer is a fixed sequence of device operations (no size crosses the host): hold it in a CUDA graph
    graph, launch = None, "eager"
    if os.environ.get("JITLLM_B200_EP_GRAPH", "1") != "0":
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    moe.forward(out, h, logits)
            launch = "one CUDA graph per layer (router, exchange, experts, exchange, combine)"
        except Exception as e:  # noqa: BLE001 -- a capture the libraries refuse falls back to eager launches
            graph, launch = None, f"eager (graph capture refused: {type(e).__name__})"
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
    ok = torch.tensor([1 if graph is not None else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if not int(ok):
        graph = None
    step = graph.replay if graph is not None else (lambda: moe.forward(out, h, logits))
    for _ in range(3):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    import bench
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with bench.ClockSampler(local) as clk:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    tt = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt)
    us = ms * 1e3 / args.steps
    hbm, burst, sustained, which = _peaks()
    wbytes_rank = epr * 3 * hidden * (ffn // 32) * 17
    line = None
    if rank == 0:
        line = ({
            "metric": "mxfp4_moe_layers_per_s", "value": 1e6 / us, "unit": "layers/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "MXFP4 codes and e8m0 scales x three e4m3 digits per activation, f32 accumulate (tcgen05 kind::mxf8f6f4.block_scale)",
            "data": "synthetic",
            "config": {"workload": "mxfp4_moe_gptoss", **MOE, "arm": "block_scaled_x3", "parallelism": f"ep{world}: {epr} experts and {ntok} tokens per rank",
                       "us_per_layer": us, "launch": launch, "exchange": "fixed capacity (tokens x top_k slots per destination, unused slots skipped by the experts)",
                       "l2": "one layer of experts per rank, re-read every step: the per-rank working set is below L2 at 8 ranks"},
            "roofline": {"bound": "hbm", "achieved": wbytes_rank / us / 1e3, "peak": hbm, "unit": "GB/s",
                         "frac": wbytes_rank / us / 1e3 / hbm, "of": which, "kernel": "whole layer incl. NCCL all-to-all, weight bytes per rank", "traffic": None},
            "e2e": None, "gpu_launches": int(per_step * args.steps), "clocks": clk.summary()})
    for h_ in hs:
        h_.free()
    dev.Close()
    dist.barrier()
    return _emit(line, emit)


def run_moe(args, emit=True):
    import torch
    from jitllm_b200 import Device, synth
    from jitllm_b200._lib import MXFP4, MoeDesc
    world, rank, local = _env()
    if world > 1:
        return run_moe_ep(args, emit)
    if rank != 0:
        return None
    torch.cuda.set_device(local)
    E, topk, hidden, ffn, ntok = MOE["E"], MOE["topk"], MOE["hidden"], MOE["ffn"], MOE["ntok"]
    rng = synth.rng_for(0xB203)
    dev = Device(local)
    dev.MoeReserve(ntok, E, topk, hidden, ffn)
    descs, keep = [], []
    for _ in range(MOE["layers"]):
        hs = [dev.Upload(MXFP4, synth.mxfp4_matrix(rng, E * r, kk), r, kk, E) for r, kk in ((ffn, hidden), (ffn, hidden), (hidden, ffn))]
        keep.append(hs)
        descs.append(MoeDesc(struct_size=C.sizeof(MoeDesc), type=MXFP4, n_expert=E, top_k=topk, hidden=hidden, ffn=ffn,
                             act=0, norm=1, scale=1.0, gate=hs[0].handle, up=hs[1].handle, down=hs[2].handle))
    h = torch.randn(ntok, hidden, device="cuda").to(torch.bfloat16)
    logits = torch.randn(ntok, E, device="cuda")
    out = torch.zeros(ntok, hidden, device="cuda")

    def run(s):
        for d in descs:
            dev.MoeDev(out, h, logits, ntok, d, None, None, s)
    run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    n0 = dev.Stats().launches
    g, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=cap):
        run(torch.cuda.current_stream().cuda_stream)
    per_replay = dev.Stats().launches - n0
    ms, clocks = _timed_replays(torch, g, args.steps, args.warmup, local)
    us = ms * 1e3 / (args.steps * MOE["layers"])
    # the two block-scaled arms on the same layers and inputs: their time, and their error against the exact arm's output
    # in the tests' parity measure (largest |difference| over max(|exact|, rms(exact)); bar 2e-3)
    from jitllm_b200._lib import MOE_ARM_BLOCK_SCALED, MOE_ARM_BLOCK_SCALED_X3
    st0 = torch.cuda.current_stream().cuda_stream
    o_exact = torch.zeros_like(out)
    dev.MoeDev(o_exact, h, logits, ntok, descs[0], None, None, st0)
    torch.cuda.synchronize()

    def other_arm(arm):
        ds = []
        for d in descs:
            b = MoeDesc.from_buffer_copy(d)
            b.arm = arm
            ds.append(b)
        o = torch.zeros_like(out)
        dev.MoeDev(o, h, logits, ntok, ds[0], None, None, st0)
        torch.cuda.synchronize()
        diff, ref = (o - o_exact).double(), o_exact.double()
        rms_ref = ref.pow(2).mean().sqrt()
        err = {"rms_rel": float(diff.pow(2).sum().sqrt() / ref.pow(2).sum().sqrt()),
               "largest_rel": float((diff.abs() / torch.maximum(ref.abs(), rms_ref)).max())}
        g2, cap2 = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.graph(g2, stream=cap2):
            for d in ds:
                dev.MoeDev(out, h, logits, ntok, d, None, None, torch.cuda.current_stream().cuda_stream)
        ms2, clocks2 = _timed_replays(torch, g2, args.steps, args.warmup, local)
        return ms2 * 1e3 / (args.steps * MOE["layers"]), ms2, clocks2, err
    us_bs, _, clocks_bs, err_bs = other_arm(MOE_ARM_BLOCK_SCALED)
    us_x3, ms_x3, clocks_x3, err_x3 = other_arm(MOE_ARM_BLOCK_SCALED_X3)
    bs_rms, bs_max = err_bs["rms_rel"], err_bs["largest_rel"]
    x3_ok = err_x3["largest_rel"] <= 2e-3          # the three-digit arm is the headline only while it is inside the bar HERE
    wbytes = E * 3 * hidden * (ffn // 32) * 17
    abytes = wbytes + ntok * hidden * 2 + ntok * E * 4 + ntok * hidden * 4
    fl = ntok * topk * 3 * 2.0 * hidden * ffn
    # end to end: the host-pointer call (activations and logits in, mixed output back; experts resident after call 1)
    hg, hu, hd = (synth.mxfp4_matrix(rng, E * ffn, hidden), synth.mxfp4_matrix(rng, E * ffn, hidden),
                  synth.mxfp4_matrix(rng, E * hidden, ffn))
    h_host = synth.to_bf16_bits(synth.activations(rng, ntok, hidden))
    lg_host = synth.activations(rng, ntok, E)
    out_host = np.zeros((ntok, hidden), np.float32)
    arm_e2e = MOE_ARM_BLOCK_SCALED_X3 if x3_ok else 0          # the headline's arm
    assert dev.MoeHost(out_host, h_host, lg_host, hg, hu, hd, E, topk, hidden, ffn, arm=arm_e2e), dev.Err()
    n_e2e = 10
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        dev.MoeHost(out_host, h_host, lg_host, hg, hu, hd, E, topk, hidden, ffn, arm=arm_e2e)
    e2e_layers = n_e2e / (time.perf_counter() - t0)
    hbm, burst, sustained, which = _peaks()
    us_exact, ms_exact, clocks_exact = us, ms, clocks
    if x3_ok:
        us, ms, clocks = us_x3, ms_x3, clocks_x3
    line = ({
        "metric": "mxfp4_moe_layers_per_s", "value": 1e6 / us, "unit": "layers/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("MXFP4 codes and e8m0 scales as they are x three e4m3 digits per activation (ue8m0 per 32), f32 accumulate "
                  "(tcgen05 kind::mxf8f6f4.block_scale)") if x3_ok else
                 "MXFP4 -> f16 (cvt e2m1x2), bf16->f16 activations, f32 accumulate (tcgen05 kind::f16)",
        "data": "synthetic",
        "config": {"workload": "mxfp4_moe_gptoss", **MOE, "us_per_layer": us, "useful_tflops": fl / us / 1e6,
                   "arm": "block_scaled_x3 (the fastest arm inside the 2e-3 parity bar in this run)" if x3_ok else "exact_f16",
                   "l2": "2 distinct layers of experts (846 MB) alternate: larger than L2"},
        "roofline": {"bound": "hbm", "achieved": abytes / us / 1e3, "peak": hbm, "unit": "GB/s", "frac": abytes / us / 1e3 / hbm,
                     "of": which, "kernel": "moe_gemm_bs_kernel<128,40,3> (gate|up, down)" if x3_ok else "moe_gemm_kernel (gate|up, down)",
                     "traffic": None, "algorithmic_bytes_per_layer": abytes},
        "arms": {
            "exact_f16": {"us_per_layer": us_exact, "hbm_frac": abytes / us_exact / 1e3 / hbm, "kernel": "moe_gemm_kernel",
                          "clocks": clocks_exact},
            "block_scaled_x3": {"us_per_layer": us_x3, "hbm_frac": abytes / us_x3 / 1e3 / hbm,
                                "kernel": "moe_gemm_bs_kernel<128,40,3>", "error_vs_exact_arm": err_x3, "inside_parity_bar": x3_ok,
                                "clocks": clocks_x3},
            "block_scaled": {"us_per_layer": us_bs, "hbm_frac": abytes / us_bs / 1e3 / hbm, "kernel": "moe_gemm_bs_kernel<64,64,1>",
                             "error_vs_exact_arm": err_bs, "inside_parity_bar": False}},
        "block_scaled_arm": {"us_per_layer": us_bs, "layers_per_s": 1e6 / us_bs, "hbm_gbs": abytes / us_bs / 1e3,
                             "hbm_frac": abytes / us_bs / 1e3 / hbm, "useful_tflops": fl / us_bs / 1e6,
                             "kernel": "moe_gemm_bs_kernel (tcgen05 kind::mxf8f6f4.block_scale; activations e4m3 + ue8m0 per 32)",
                             "weights_by_tma": bool(dev.lib.jl_moe_bs_weights_by_tma(dev.ctx)),
                             "error_vs_exact_arm": {"rms_rel": bs_rms, "largest_rel": bs_max,
                                                    "note": "outside the 2e-3 parity bar by construction; selected only by jl_moe_desc.arm"},
                             "clocks": clocks_bs},
        "e2e": {"value": e2e_layers, "unit": "layers/s", "h2d_bytes_per_step": ntok * hidden * 2 + ntok * E * 4,
                "d2h_bytes_per_step": ntok * hidden * 4, "note": "jl_moe host-pointer call, wall clock"},
        "gpu_launches": int(per_replay * args.steps), "clocks": clocks})
    for hs in keep:
        for h_ in hs:
            h_.free()
    dev.Close()
    return _emit(line, emit)


# ------------------------------------------------------------------ decoder
def run_decode(args, emit=True, batches=None, steps=None):
    """Llama-3-8B-shaped Q4_K decoder: prompt prefill (GEMM path), then greedy decode steps replayed from a CUDA
    graph. Batch 1 runs the block kernel (one persistent launch per token); larger batches the per-matmul chain.
    Under torchrun the model is tensor-parallel over the ranks (strong scaling: one model, N GPUs): at batch 1 the
    ranks exchange partial sums inside the kernel over peer slots, above it through NCCL all-reduce.
    Returns one line per batch size."""
    import torch
    import bench
    from jitllm_b200 import Device
    from jitllm_b200.decoder import Config, Decoder
    world, rank, local = _env()
    torch.cuda.set_device(local)
    dist = _pg(local) if world > 1 else None
    batches = batches or [args.batch]
    T = args.prompt
    steps = steps or args.steps
    warm = max(args.warmup, 3)
    dev = Device(local)
    dec = Decoder(dev, Config(), max_batch=max(batches), max_len=T + len(batches) * (warm + steps + 24) + 16, rank=rank,
                  world=world, max_prefill=T, group=dist.group.WORLD if world > 1 else None)
    prompt = torch.randint(0, 128256, (T,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
    hbm, burst, sustained, which = _peaks()
    wb = dec.weight_bytes                                       # per rank
    lines = []
    with torch.no_grad():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        nxt = dec.prefill(prompt)
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        use_block = 1 in batches and dec.prep_block_kernel()
        start = T
        for B in batches:
            block = use_block and B == 1
            tok = nxt.expand(B).contiguous()
            pos = torch.tensor([start], device="cuda")

            def one_step():
                if block:
                    out = dec.decode_step_block(tok, pos, advance=world == 1)
                    if world > 1:
                        tok.copy_(out)
                        pos.add_(1)
                else:
                    out = dec.decode_step(tok, pos)
                    tok.copy_(out)
                    pos.add_(1)
            for _ in range(2):
                one_step()                                     # eager warm-up (sizes the attention scratch)
            torch.cuda.synchronize()
            n0 = dev.Stats().launches
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step()
            lib_launches = dev.Stats().launches - n0
            aux_launches = 0 if block else 1 + 6 * dec.cfg.n_layer + 1   # norms, rope, attention, silu per layer; first norm; argmax
            if block and world > 1:
                aux_launches = 1                                # argmax over the gathered vocabulary shards
            for _ in range(warm):
                g.replay()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with bench.ClockSampler(local) as clk:
                e0.record()
                for _ in range(steps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            ok = dev.StatusPoll()
            # end to end: the token ids cross the host boundary every step (ids in from pinned memory, next ids out)
            tok_pin = torch.empty(B, dtype=torch.int64).pin_memory()
            tok_pin.copy_(tok)
            n_e2e = min(steps, 16)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n_e2e):
                tok.copy_(tok_pin, non_blocking=True)
                g.replay()
                tok_pin.copy_(tok, non_blocking=True)
                torch.cuda.synchronize()
            e2e_s = time.perf_counter() - t0
            start = int(pos.item()) + 1
            if world > 1:
                tt = torch.tensor([ms, e2e_s, 0.0 if ok else 1.0], device="cuda", dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms, e2e_s, ok = float(tt[0]), float(tt[1]), float(tt[2]) == 0.0
            if not ok:
                raise RuntimeError("a bounded device-side wait ran out during the timed decode steps: " + dev.Err())
            ms_step = ms / steps
            kv_bytes = B * 2 * (start - 1) * dec.hkv * dec.cfg.head_dim * 2 * dec.cfg.n_layer   # K and V rows read per step, per rank
            line = {
                "metric": "decode_tok_s", "value": B * 1e3 / ms_step, "unit": "tok/s", "n_gpus": world, "steps": steps,
                "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "Q4_K weights, f32 activations (int8-digit MMA decode / f16 tcgen05 GEMM), bf16 KV",
                "data": "synthetic (random-init Q4_K weights, random prompt ids)",
                "config": {"workload": "llama8b_q4k_decode", "batch": B, "prompt": T, "layers": 32, "hidden": 4096, "heads": "32q/8kv x128",
                           "ffn": 14336, "vocab": 128256, "parallelism": f"tp{world}", "prefill_tok_s": T / prefill_s,
                           "form": ("block kernel: one persistent launch per token" + (", partial sums exchanged in-kernel over peer slots" if world > 1 else ""))
                                   if block else ("per-matmul chain" + (", NCCL all-reduce" if world > 1 else "")),
                           "l2": f"weights per rank {wb / 1e9:.2f} GB stream every step: larger than L2",
                           "weight_roofline_tok_s": B * hbm * 1e9 / wb},
                "roofline": {"bound": "hbm", "achieved": (wb + kv_bytes) / ms_step / 1e6, "peak": hbm, "unit": "GB/s",
                             "frac": (wb + kv_bytes) / ms_step / 1e6 / hbm, "of": which,
                             "kernel": "jl_block_kernel" if block else "whole decode step",
                             "algorithmic_bytes_per_step": wb + kv_bytes, "traffic": None},
                "e2e": {"value": B * n_e2e / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8,
                        "note": "token ids in from pinned host memory and next ids back to the host every step, wall clock"},
                "gpu_launches": int((lib_launches + aux_launches) * steps), "clocks": clk.summary()}
            del g
            torch.cuda.synchronize()
            if rank == 0:
                lines.append(_emit(line, emit))
    if use_block:
        dec.block.free()
    del dec
    dev.Close()
    if world > 1:
        dist.barrier()
    return lines


# ------------------------------------------------------------------ sharded forms against the unsharded ones
def profile_case(args):
    """Small fixed cases for a profiler to capture: no timing, few launches, a few hundred MB on the device (but
    above the 126 MB L2, so DRAM counters mean something). Prints the kernels' launch count."""
    import torch
    from jitllm_b200 import Q4_K, Q8_0, Device, synth
    from jitllm_b200 import _lib
    torch.cuda.set_device(0)
    case = args.profile
    stream = torch.cuda.current_stream().cuda_stream
    rng = synth.rng_for(0x9F0)
    forms = {"auto": 0, "split": _lib.FORM_SPLIT, "fused": _lib.FORM_FUSED, "wide": _lib.FORM_WIDE, "l1": _lib.FORM_L1}
    if case in ("gemv", "q8"):
        t, ntok = (Q4_K, 1) if case == "gemv" else (Q8_0, 32)
        n = k = 4096
        ring = 32 if case == "gemv" else 16
        flags = _lib.FLAG_DECODE_CONCURRENT if args.form == "concurrent" else 0
        with Device(0, decode_form=forms.get(args.form, 0), flags=flags) as dev:
            dev.Reserve(n, k, ntok)
            ws = [dev.Upload(t, synth.matrix(rng, t, n, k), n, k) for _ in range(ring)]
            x = torch.randn(ntok, k, device="cuda")
            y = torch.empty(ntok, n, device="cuda")
            for i in range(ring + 8):
                dev.MatMulDev(y, ws[i % ring], x, ntok, stream)
            torch.cuda.synchronize()
            assert dev.StatusPoll(), dev.Err()
            print(json.dumps({"profile": case, "form": args.form, "launches": dev.Stats().launches}))
            for w in ws:
                w.free()
    elif case == "gemm":
        n, k, ntok = 14336, 4096, 512
        with Device(0) as dev:
            dev.Reserve(n, k, ntok)
            ws = [dev.Upload(Q4_K, synth.q4k_matrix(rng, n, k), n, k) for _ in range(4)]
            x = torch.randn(ntok, k, device="cuda").to(torch.bfloat16)
            y = torch.empty(ntok, n, device="cuda", dtype=torch.bfloat16)
            for i in range(6):
                dev.MatMulDev(y, ws[i % 4], x, ntok, stream)
            torch.cuda.synchronize()
            assert dev.StatusPoll(), dev.Err()
            print(json.dumps({"profile": case, "launches": dev.Stats().launches}))
    elif case == "moe":
        a2 = type(args)(**{**vars(args), "steps": 2, "warmup": 1})
        run_moe(a2, emit=True)
    elif case == "block":
        from jitllm_b200.decoder import Config, Decoder
        T = 2048
        with Device(0) as dev:
            dec = Decoder(dev, Config(n_layer=4, vocab=32768), max_batch=1, max_len=T + 32, max_prefill=64, seed=5)
            assert dec.prep_block_kernel(), dev.Err()
            g = torch.Generator(device="cuda").manual_seed(1)
            dec.k_cache[:, :, :, :T] = torch.randn(dec.k_cache[:, :, :, :T].shape, device="cuda", generator=g).to(torch.bfloat16)
            dec.v_cache[:, :, :, :T] = torch.randn(dec.v_cache[:, :, :, :T].shape, device="cuda", generator=g).to(torch.bfloat16)
            tok, pos = torch.tensor([17], device="cuda"), torch.tensor([T], device="cuda")
            with torch.no_grad():
                for _ in range(6):
                    dec.decode_step_block(tok, pos, advance=True)
            torch.cuda.synchronize()
            assert dev.StatusPoll(), dev.Err()
            print(json.dumps({"profile": case, "layers": 4, "cached": T, "steps": 6, "last_token": int(tok)}))
            dec.block.free()
    elif case == "attn":
        L = _lib.load()
        n, hq, hkv, d, pos = 1, 32, 8, 128, 2048
        max_len = pos + 16
        g = torch.Generator(device="cuda").manual_seed(3)
        q = torch.randn(n, hq, d, device="cuda", generator=g).to(torch.bfloat16)
        caches = [(torch.randn(n, hkv, max_len, d, device="cuda", generator=g).to(torch.bfloat16),
                   torch.randn(n, hkv, max_len, d, device="cuda", generator=g).to(torch.bfloat16)) for _ in range(24)]   # 24 x 8.4 MB > L2
        scr = torch.zeros(L.jl_aux_attn_scratch_bytes(n, hq, hkv, max_len), device="cuda", dtype=torch.uint8)
        pd = torch.tensor([pos], device="cuda")
        out = torch.empty(n, hq * d, device="cuda")
        for kc, vc in caches:
            assert L.jl_aux_attn_decode(out.data_ptr(), None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pd.data_ptr(), scr.data_ptr(),
                                        n, hq, hkv, d, max_len, stream) == 0
        torch.cuda.synchronize()
        print(json.dumps({"profile": case, "launches": len(caches)}))
    else:
        raise SystemExit(f"unknown profile case {case}")


def _perr(got, ref):
    """max_i |got - ref| / max(|ref_i|, rms(ref)): the output-parity measure (bar 2e-3)."""
    got, ref = got.double().reshape(-1), ref.double().reshape(-1)
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    return float(((got - ref).abs() / ref.abs().clamp_min(rms)).max())


def sharded_parity(local):
    """Run on the live process group before anything is timed: (1) one full-width Llama-3-8B-shaped block + head,
    tensor-parallel over the ranks, against the same block unsharded on this rank's own GPU -- batch 1 through the
    block kernel (partial sums exchanged in-kernel over peer slots) and batch 2 through the per-matmul chain (NCCL
    all-reduce); (2) a mixture layer expert-parallel over the ranks against the whole layer on one GPU. The
    unsharded forms are what the single-GPU parity tests hold against the CPU oracle. Returns the two errors."""
    import torch
    import torch.distributed as dist
    from jitllm_b200 import Device, parallel, synth
    from jitllm_b200._lib import MOE_ARM_BLOCK_SCALED_X3, MXFP4, MoeDesc
    from jitllm_b200.decoder import Config, Decoder
    world, rank, _ = _env()
    dev = Device(local)
    T = 200
    tp_err = 0.0
    with torch.no_grad():
        cfg = Config(n_layer=1, vocab=8192)
        one = Decoder(dev, cfg, max_batch=2, max_len=T + 8, max_prefill=16, share_full=True, seed=5)
        tp = Decoder(dev, cfg, max_batch=2, max_len=T + 8, max_prefill=16, share_full=True, seed=5, rank=rank, world=world)
        g = torch.Generator(device="cuda").manual_seed(3)                  # the same cache contents on every rank
        kfull = torch.randn(1, 2, cfg.n_kv, T, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)
        vfull = torch.randn(1, 2, cfg.n_kv, T, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)
        one.k_cache[:, :, :, :T], one.v_cache[:, :, :, :T] = kfull, vfull
        tp.k_cache[:, :, :, :T] = kfull[:, :, rank * tp.hkv:(rank + 1) * tp.hkv]
        tp.v_cache[:, :, :, :T] = vfull[:, :, rank * tp.hkv:(rank + 1) * tp.hkv]
        ok = one.prep_block_kernel() and tp.prep_block_kernel()
        if not ok:
            raise RuntimeError("the block kernel declined the Llama-3-8B-shaped block: " + dev.Err())
        pos = torch.tensor([T], device="cuda")
        for B in (1, 2):
            tok = torch.tensor([17, 4099][:B], device="cuda")
            if B == 1:
                one.decode_step_block(tok.clone(), pos)
            else:
                one.decode_step(tok, pos)
            ref = one.last_logits.clone()
            if B == 1:
                tp.decode_step_block(tok.clone(), pos)
            else:
                tp.decode_step(tok, pos)
            parts = [torch.empty_like(tp.last_logits) for _ in range(world)]
            dist.all_gather(parts, tp.last_logits.contiguous())
            torch.cuda.synchronize()
            if not dev.StatusPoll():
                raise RuntimeError("tensor-parallel step: " + dev.Err())
            tp_err = max(tp_err, _perr(torch.cat(parts, dim=-1), ref))
        one.block.free()
        tp.block.free()
        del one, tp
        # ---- expert parallel
        E, topk, hidden, ffn, ntok = 32, 4, 576, 576, 64
        rng = synth.rng_for(0xE9)                                          # the same banks on every rank
        banks = [synth.mxfp4_matrix(rng, E * r, kk) for r, kk in ((ffn, hidden), (ffn, hidden), (hidden, ffn))]
        epr = E // world
        stream = torch.cuda.current_stream().cuda_stream
        full = [dev.Upload(MXFP4, b, r, kk, E) for b, (r, kk) in zip(banks, ((ffn, hidden), (ffn, hidden), (hidden, ffn)))]
        mine = [dev.Upload(MXFP4, parallel.shard_experts(b, MXFP4, E, r, kk, rank, world)[0], r, kk, epr)
                for b, (r, kk) in zip(banks, ((ffn, hidden), (ffn, hidden), (hidden, ffn)))]
        dev.MoeReserve(world * ntok * topk, E, topk, hidden, ffn)
        d_full = MoeDesc(struct_size=C.sizeof(MoeDesc), type=MXFP4, n_expert=E, top_k=topk, hidden=hidden, ffn=ffn, act=0, norm=1,
                         scale=1.0, gate=full[0].handle, up=full[1].handle, down=full[2].handle)
        d_local = MoeDesc(struct_size=C.sizeof(MoeDesc), type=MXFP4, n_expert=epr, top_k=1, hidden=hidden, ffn=ffn, act=0, norm=1,
                          scale=1.0, gate=mine[0].handle, up=mine[1].handle, down=mine[2].handle,
                          arm=MOE_ARM_BLOCK_SCALED_X3)      # the arm the sharded bench runs; the unsharded side is the exact arm
        g = torch.Generator(device="cuda").manual_seed(100 + rank)          # every rank routes its own tokens
        h = (torch.randn(ntok, hidden, device="cuda", generator=g) * 0.25).to(torch.bfloat16)
        logits = torch.randn(ntok, E, device="cuda", generator=g)
        ref = torch.zeros(ntok, hidden, device="cuda")
        dev.MoeDev(ref, h, logits, ntok, d_full, None, None, stream)

        def route(lg):
            sel = torch.empty(lg.shape[0], topk, dtype=torch.int32, device="cuda")
            wt = torch.empty(lg.shape[0], topk, dtype=torch.float32, device="cuda")
            dev.MoeRouteDev(lg, lg.shape[0], d_full, sel, wt, torch.cuda.current_stream().cuda_stream)
            return sel, wt

        def experts(rows, ids):
            y = torch.empty(rows.shape[0], hidden, dtype=torch.float32, device="cuda")
            dev.MoeExpertsDev(y, rows.contiguous(), ids.contiguous(), rows.shape[0], d_local, torch.cuda.current_stream().cuda_stream)
            return y
        out = torch.zeros(ntok, hidden, device="cuda")
        parallel.ExpertParallelMoE(route, experts, E, topk, hidden).forward(out, h, logits)
        torch.cuda.synchronize()
        ep_err = _perr(out, ref)
        for w in full + mine:
            w.free()
    dev.Close()
    tt = torch.tensor([tp_err, ep_err], device="cuda", dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    return {"tp_err": float(tt[0]), "ep_err": float(tt[1]), "bar": 2e-3,
            "against": "the unsharded forms on one GPU (which the single-GPU tests hold against the CPU oracle)"}


# ------------------------------------------------------------------ reference arm (CPU restatement, host cores)
def run_reference(args):
    """The reference's CPU path for the same workloads: its int8-activation integer-dot arithmetic for the dense
    matmuls, its expert-major mixture layer for the MoE, restated in oracle/jl_oracle.c (the reference is Go and
    cannot be built here). Every step is a bounded sample of the workload, stated in `sample`."""
    import oracle
    from jitllm_b200 import synth
    from jitllm_b200._lib import MXFP4, Q4_K
    world, rank, local = _env()
    if rank != 0:
        return
    oracle.build()
    cores = os.cpu_count() or 1
    name = args.workload
    rng = synth.rng_for(0xB2FF)

    def timed(step):
        for _ in range(args.warmup):
            step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        return (time.perf_counter() - t0) / args.steps

    if name == "q4k_gemm_prefill":
        nrows, k, ntok = 14336, 4096, 64
        w, x = synth.q4k_matrix(rng, nrows, k), synth.activations(rng, ntok, k)
        dt = timed(lambda: oracle.matmul_int8(Q4_K, w, x, nrows, k, ntok, window=256, nthreads=cores))
        metric, unit, val = "q4k_gemm_tflops", "TFLOP/s", 2.0 * ntok * nrows * k / dt / 1e12
        sample = f"step = one {ntok}-token slice of the 512x{nrows}x{k} GEMM, {cores} threads"
    elif name == "q8_0_batch32":
        from jitllm_b200._lib import Q8_0
        ws = [synth.q8_0_matrix(rng, r, kk) for r, kk in Q8_SHAPES]
        xs = [synth.activations(rng, Q8_NTOK, kk) for _, kk in Q8_SHAPES]

        def q8step():
            for (r, kk), w, x in zip(Q8_SHAPES, ws, xs):
                oracle.matmul_int8(Q8_0, w, x, r, kk, Q8_NTOK, window=32, nthreads=cores)
        dt = timed(q8step)
        nbytes = sum(r * kk * 34 // 32 + Q8_NTOK * (kk + r) * 4 for r, kk in Q8_SHAPES)
        metric, unit, val = "q8_0_batch32_gbs", "GB/s", nbytes / dt / 1e9
        sample = f"step = the three batch-32 matmuls once each (one weight copy per shape), {cores} threads"
    elif name == "mxfp4_moe_gptoss":
        E, topk, hidden, ffn, ntok = MOE["E"], MOE["topk"], MOE["hidden"], MOE["ffn"], 16
        g, u, d = (synth.mxfp4_matrix(rng, E * ffn, hidden), synth.mxfp4_matrix(rng, E * ffn, hidden),
                   synth.mxfp4_matrix(rng, E * hidden, ffn))
        h, lg = synth.activations(rng, ntok, hidden), synth.activations(rng, ntok, E)
        sel, wt = np.zeros((ntok, topk), np.int32), np.zeros((ntok, topk), np.float32)
        for i in range(ntok):
            s_, _, w_, _, _ = oracle.moe_router(oracle.softmax(lg[i]), topk)
            sel[i], wt[i] = s_, w_
        dt = timed(lambda: oracle.moe_layer(h, MXFP4, g, u, d, sel, wt, E, hidden, ffn, nthreads=cores))
        metric, unit, val = "mxfp4_moe_layers_per_s", "layers/s", (ntok / MOE["ntok"]) / dt
        sample = f"step = {ntok} of the layer's {MOE['ntok']} tokens (rate scaled by {ntok}/{MOE['ntok']}), {cores} threads"
    else:
        shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
        ws = [synth.q4k_matrix(rng, r, kk) for r, kk in shapes]
        xs = [synth.activations(rng, args.batch, kk) for _, kk in shapes]

        def layer():
            for (r, kk), w, x in zip(shapes, ws, xs):
                oracle.matmul_int8(Q4_K, w, x, r, kk, args.batch, window=256, nthreads=cores)
        dt = timed(layer)
        head = 128256 * 4096 / sum(r * kk for r, kk in shapes)      # lm_head in units of one layer's weights
        metric, unit, val = "decode_tok_s", "tok/s", args.batch / (dt * (32 + head))
        sample = (f"step = the four matmuls of ONE layer at batch {args.batch}; tok/s = batch / (32 + {head:.2f}) layer times "
                  f"(matmuls only: attention, norms and sampling are not timed), {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 activations x quantized weights -> f32", "data": "synthetic",
        "config": {"workload": name, "note": "CPU restatement of the reference's arithmetic (oracle/jl_oracle.c)"},
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}), flush=True)
