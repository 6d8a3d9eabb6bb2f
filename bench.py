"""Benchmark of the NF4-LoRA hot path.

    python bench.py --gpus 1 --steps 20 --warmup 5                       # this repository's CUDA path
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference --steps 3 --warmup 1                # the reference's eager path on host cores

One "step" is one forward + backward of a frozen NF4 linear with its LoRA adapter on one batch of tokens.
Workload (BASELINE config 2's weight, at the M the targets are quoted for): W [14336, 4096] ~ N(0, 0.02),
NF4 blocksize 64 with the absmax double-quantised to 8 bit in blocks of 256, LoRA r=16 alpha=32,
M = 4096 tokens per GPU, X and dY ~ N(0, 1) in bf16, seeded synthetic data.  With N > 1 GPUs the token batch is
sharded (4096 tokens per GPU, weak scaling) and the LoRA gradients are all-reduced over NCCL every step, on a side
stream that overlaps the next step.  The same line also carries, at every N, the second half of the metric: training
targets per second of a full QLoRA step at BASELINE config 4's shapes (``extra.qlora_step_c4``).
Prints exactly one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

N_OUT, K_IN, RANK, ALPHA, M_PER_GPU = 14336, 4096, 16, 32.0, 4096
SCALING = ALPHA / RANK
# dram__bytes_read.sum + dram__bytes_write.sum of one backward GEMM launch at M = 4096 (238.5 MB + 23.6 MB, the fp32
# partial tiles of the split last wave included), taken from an ncu --set full capture of `bench.py --profile gemm_bwd`;
# the summary of that capture sits under profiles/.
GEMM_BWD_DRAM_BYTES_PER_LAUNCH = 262.1e6
METRIC = "nf4_lora_linear_fwd_bwd_tflops"
WORKLOAD = ("NF4-LoRA linear fwd+bwd, W[14336,4096] NF4 bs64 double-quant absmax, r=16 alpha=32, "
            "M=4096 tokens per GPU, bf16")


def linear_flops(m: int, n: int = N_OUT, k: int = K_IN, r: int = RANK, backward: bool = True) -> float:
    """Algorithmic FLOPs: fwd 2MNK + 2Mr(K+N); fwd+bwd 4MNK + 6Mr(K+N) (recomputation not counted)."""
    return (4.0 if backward else 2.0) * m * n * k + (6.0 if backward else 2.0) * m * r * (k + n)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"bf16_tflops": float(data["bf16_tflops"]), "bf16_tflops_sustained": float(data["bf16_tflops_sustained"]),
                "hbm_gbs": float(data["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            handle = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = handle.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=handle, stderr=subprocess.DEVNULL)
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        clocks, reasons, sm_max = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                sm_max = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if clocks:
            clocks.sort()
            busy = clocks[len(clocks) // 2:]  # upper half = samples under load
            out["sm_mhz"] = busy[len(busy) // 2]
            out["sm_max_mhz"] = sm_max
            out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------------------------------------------
# reference arm: the reference's eager CPU path (oracle restatement) on the host cores
# ------------------------------------------------------------------------------------------------------

def synthetic_quantized_weight_cpu(n: int, k: int, seed: int):
    """Seeded synthetic NF4 weight made directly on the host (nearest level through the midpoints of the
    codebook; ties do not matter for timing)."""
    from oracle import molt_oracle as oracle

    gen = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=gen) * 0.02
    blocks = w.reshape(-1, 64)
    scales = blocks.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
    mids = (oracle.NF4_CODEBOOK[1:] + oracle.NF4_CODEBOOK[:-1]) / 2
    codes = torch.bucketize(blocks / scales[:, None], mids).to(torch.uint8)
    packed = ((codes[:, 0::2] << 4) | codes[:, 1::2]).reshape(-1)
    q = oracle.OracleNF4(packed, scales, (n, k), 64, n * k, oracle.HIGH_FIRST)
    nested = oracle.nest_absmax(scales)
    return q, oracle.resolve_nested_absmax(nested)


def time_cpu_reference(sample_rows: int, steps: int, warmup: int, q=None, scales=None):
    """Times dequantise + forward + backward (which dequantises again) exactly as the reference's eager path does."""
    from oracle import molt_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if q is None:
        q, scales = synthetic_quantized_weight_cpu(N_OUT, K_IN, 1337)
    gen = torch.Generator().manual_seed(1340)
    a = torch.randn(RANK, K_IN, generator=gen) * 0.01
    b = torch.randn(N_OUT, RANK, generator=gen) * 0.01
    x = torch.randn(sample_rows, K_IN, generator=gen)
    dy = torch.randn(sample_rows, N_OUT, generator=gen)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.nf4_lora_fwd_bwd(q, x, dy, a, b, SCALING, scales)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    seconds = sum(times) / len(times)
    what = "the full workload" if sample_rows == M_PER_GPU else f"{sample_rows} of {M_PER_GPU} token rows per step"
    return {"value": linear_flops(sample_rows) / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{what}: {sample_rows} token rows, full weight, fp32, torch {torch.__version__} "
                      f"on {cores} host threads; {steps} timed steps",
            "ms_per_step": seconds * 1e3}


def time_cpu_config1(steps: int = 10, warmup: int = 3):
    """BASELINE config 1 on the host cores through the oracle's statement of the reference's eager path
    (NF4Tensor.quantize once, untimed; then dequantise + forward + backward, which dequantises again)."""
    from oracle import molt_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n, k, m, r = 4864, 896, 512, 16
    w, a, b, x, dy = oracle.seeded_linear_case(n, k, m, r, seed=1337)
    q = oracle.nf4_quantize(w, 64)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.nf4_lora_fwd_bwd(q, x, dy, a, b, 2.0)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    seconds = sum(times) / len(times)
    return {"workload": "BASELINE config 1: W[4864,896] NF4 bs64 fp32 absmax, r=16, M=512, fp32 on CPU",
            "ms_per_step": seconds * 1e3, "gflops": linear_flops(m, n, k, r) / seconds / 1e9, "cores": cores,
            "kind": "port"}


def run_reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    base = time_cpu_reference(M_PER_GPU, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": M_PER_GPU, "n": N_OUT, "k": K_IN, "rank": RANK},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------------------

def event_time_ms(fn, iters: int, warmup: int = 0) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def graph_time_ms(calls, replays: int = 20) -> float:
    """Device time per call for short kernels: the calls (one per rotating buffer set) are captured into a
    CUDA graph so that host launch overhead is not what is measured; returns ms per call."""
    for fn in calls:
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for fn in calls:
            fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / (replays * len(calls))


def run_ours(args) -> int:
    import torch.distributed as dist

    from molt_b200 import _native
    from molt_b200.methods import QuantState, quantize_nf4, resolved_nf4_scales, scheduled_nf4_lora
    from molt_b200.methods._linear import weight_desc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")   # keeps NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
    lib = _native.library()
    peaks = measured_peaks()

    # ---- synthetic workload (seeded; identical weight on every rank, different tokens per rank) ----
    gen = torch.Generator(device=device).manual_seed(1337)
    w = torch.randn(N_OUT, K_IN, device=device, generator=gen) * 0.02
    packed, state = quantize_nf4(w, 64, compress_statistics=True)
    del w
    lora_a = torch.randn(RANK, K_IN, device=device, generator=gen) * 0.01
    lora_b = torch.randn(N_OUT, RANK, device=device, generator=gen) * 0.01
    tok_gen = torch.Generator(device=device).manual_seed(4242 + rank)
    m = M_PER_GPU
    x = torch.randn(m, K_IN, device=device, generator=tok_gen).bfloat16()
    dy = torch.randn(m, N_OUT, device=device, generator=tok_gen).bfloat16()
    desc = weight_desc(packed, state)

    y = torch.empty(m, N_OUT, device=device, dtype=torch.bfloat16)
    dx = torch.empty(m, K_IN, device=device, dtype=torch.bfloat16)
    t_buf = torch.empty(m, 64, device=device, dtype=torch.bfloat16)
    grads = torch.zeros(RANK * K_IN + N_OUT * RANK, device=device, dtype=torch.float32)
    da, db = grads[: RANK * K_IN].view(RANK, K_IN), grads[RANK * K_IN:].view(N_OUT, RANK)
    ws_bytes = max(lib.molt_workspace_bytes(_native.OP_LORA_FWD, m, N_OUT, K_IN, RANK),
                   lib.molt_workspace_bytes(_native.OP_LORA_BWD, m, N_OUT, K_IN, RANK))
    ws = torch.empty(ws_bytes, device=device, dtype=torch.uint8)
    stream = _native.stream_handle(device)

    # Two gradient buffers: the all-reduce of step i runs on a side stream while step i + 1 computes into the other one.
    grad_sets = [(grads, da, db)]
    if world > 1:
        more = torch.zeros_like(grads)
        grad_sets.append((more, more[: RANK * K_IN].view(RANK, K_IN), more[RANK * K_IN:].view(N_OUT, RANK)))
    comm_stream = torch.cuda.Stream(device=device) if world > 1 else None
    reduced = [torch.cuda.Event() for _ in grad_sets]
    main = torch.cuda.current_stream(device)
    counter = [0]

    def step_device():
        flat, ga, gb = grad_sets[counter[0] % len(grad_sets)]
        slot = counter[0] % len(grad_sets)
        counter[0] += 1
        if world > 1:
            main.wait_event(reduced[slot])          # the collective that last read this buffer is done
        _native.check(lib.molt_nf4_lora_fwd(ctypes.byref(desc), x.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
                                            SCALING, RANK, y.data_ptr(), m, t_buf.data_ptr(), ws.data_ptr(), ws_bytes,
                                            _native.PATH_AUTO, stream))
        _native.check(lib.molt_nf4_lora_bwd(ctypes.byref(desc), x.data_ptr(), dy.data_ptr(), lora_a.data_ptr(),
                                            lora_b.data_ptr(), SCALING, RANK, dx.data_ptr(), ga.data_ptr(),
                                            gb.data_ptr(), m, t_buf.data_ptr(), 0, ws.data_ptr(), ws_bytes,
                                            _native.PATH_AUTO, stream))
        if world > 1:
            comm_stream.wait_stream(main)
            with torch.cuda.stream(comm_stream):
                dist.all_reduce(flat, op=dist.ReduceOp.SUM)
                reduced[slot].record(comm_stream)

    def drain():
        if world > 1:
            main.wait_stream(comm_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def check_status(where):
        status = _native.read_status(device)
        if status:
            raise SystemExit(f"a bounded device wait expired during {where} (status 0x{status:08x})")

    if args.profile:
        return profile_case(args.profile, lib, device, desc, packed, state, lora_a, lora_b, x, dy, y, dx, ws, ws_bytes)

    # ---- timed region: device-resident inputs -------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step_device()
    drain()
    barrier()
    launches_before = lib.molt_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        start.record()
        for _ in range(args.steps):
            step_device()
        drain()
        stop.record()
        barrier()
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    elapsed_ms = float(elapsed_ms.item())
    launches = int(lib.molt_launch_count() - launches_before)
    check_status("the timed region")
    clocks = sampler.summary()
    ms_per_step = elapsed_ms / args.steps
    value = world * linear_flops(m) / (ms_per_step * 1e-3) / 1e12

    # ---- the same step for about 1.5 s without a pause: what the chip sustains under its power cap ----------
    sustained_steps = max(args.steps, int(1500.0 / ms_per_step))
    with ClockSampler(local_rank) as sustained_sampler:
        barrier()
        start.record()
        for _ in range(sustained_steps):
            step_device()
        drain()
        stop.record()
        barrier()
    sustained_ms = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(sustained_ms, op=dist.ReduceOp.MAX)
    sustained_ms = float(sustained_ms.item())
    check_status("the sustained run")
    sustained_value = world * linear_flops(m) * sustained_steps / (sustained_ms * 1e-3) / 1e12
    sustained = {"steps": sustained_steps, "seconds": sustained_ms * 1e-3, "value": sustained_value, "unit": "TFLOP/s",
                 "ms_per_step": sustained_ms / sustained_steps,
                 "frac_of_bf16_burst_peak": sustained_value / world / peaks["bf16_tflops"],
                 "frac_of_bf16_sustained_peak": sustained_value / world / peaks["bf16_tflops_sustained"],
                 "clocks": sustained_sampler.summary()}

    # ---- end to end through the Python API, host buffers, copies inside the timed region -------------
    x_host = x.cpu().pin_memory()
    dy_host = dy.cpu().pin_memory()
    grads_host = torch.empty(grads.shape, dtype=torch.float32).pin_memory()
    a_param = lora_a.clone().requires_grad_()
    b_param = lora_b.clone().requires_grad_()
    # Two device buffers per input and a copy stream: the copy of step i+1's inputs runs while step i computes, and the
    # gradients of step i go back to the host behind it.  Every step still copies its own inputs in and its result out.
    x_dev = [torch.empty_like(x) for _ in range(2)]
    dy_dev = [torch.empty_like(dy) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=device)
    copied = [torch.cuda.Event() for _ in range(2)]     # inputs of a slot are on the device
    consumed = [torch.cuda.Event() for _ in range(2)]   # the step that used a slot has finished with it
    main_stream = torch.cuda.current_stream(device)

    def stage_inputs(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            x_dev[slot].copy_(x_host, non_blocking=True)
            dy_dev[slot].copy_(dy_host, non_blocking=True)
            copied[slot].record(copy_stream)

    def step_e2e(slot):
        stage_inputs(slot ^ 1)                   # next step's inputs, overlapped with this step's kernels
        main_stream.wait_event(copied[slot])
        a_param.grad = None
        b_param.grad = None
        xin = x_dev[slot].detach().requires_grad_()
        out = scheduled_nf4_lora(xin, packed, a_param, b_param, state, SCALING)
        out.backward(dy_dev[slot])
        consumed[slot].record(main_stream)
        flat = torch.cat([a_param.grad.reshape(-1), b_param.grad.reshape(-1)])
        if world > 1:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        grads_host.copy_(flat, non_blocking=True)

    e2e_steps = max(4, min(args.steps, 10))
    for slot in range(2):
        consumed[slot].record(main_stream)
    stage_inputs(0)
    for i in range(4):
        step_e2e(i & 1)
    barrier()
    start.record()
    for i in range(e2e_steps):
        step_e2e(i & 1)
    stop.record()
    barrier()
    e2e_ms = torch.tensor([start.elapsed_time(stop) / e2e_steps], device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    check_status("the end-to-end run")
    # what bounds it: the same host-to-device copies alone, all ranks at once (they share the host's memory and PCIe fabric)
    h2d_bytes = x_host.numel() * 2 + dy_host.numel() * 2
    barrier()
    start.record()
    for i in range(e2e_steps):
        x_dev[i & 1].copy_(x_host, non_blocking=True)
        dy_dev[i & 1].copy_(dy_host, non_blocking=True)
    stop.record()
    barrier()
    copy_ms = torch.tensor([start.elapsed_time(stop) / e2e_steps], device=device)
    if world > 1:
        dist.all_reduce(copy_ms, op=dist.ReduceOp.MAX)
    copy_ms = float(copy_ms.item())
    e2e_value = world * linear_flops(m) / (float(e2e_ms.item()) * 1e-3) / 1e12
    e2e = {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": float(e2e_ms.item()),
           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": grads_host.numel() * 4,
           "pipelining": "inputs of step i+1 are copied on a second stream while step i computes",
           "h2d_copies_alone_ms_per_step": copy_ms, "h2d_gbs_per_gpu_alone": h2d_bytes / copy_ms / 1e6,
           "bound": ("host-to-device copies: alone, with all ranks copying at once, they take "
                     f"{copy_ms:.2f} ms per step against {ms_per_step:.2f} ms of kernels"
                     if copy_ms > ms_per_step else "kernels")}
    del x_dev, dy_dev, x_host, dy_host

    # ---- roofline of the dominant kernel: the tcgen05 GEMM, timed alone with CUDA events ---------------
    plain_state = QuantState(absmax=resolved_nf4_scales(state), shape=(N_OUT, K_IN), nibble_order=state.nibble_order)
    plain_desc = weight_desc(packed, plain_state)

    def gemm_only():  # exactly one launch of the backward GEMM (+ its fix-up): dx = dy . deq(W)
        _native.check(lib.molt_nf4_dx(ctypes.byref(plain_desc), dy.data_ptr(), None, None, 0, 0.0, 0, dx.data_ptr(), m,
                                      ws.data_ptr(), ws_bytes, _native.PATH_TCGEN05, stream))

    gemm_ms = event_time_ms(gemm_only, iters=max(5, args.steps), warmup=3)
    check_status("the roofline run")
    achieved = 2.0 * m * N_OUT * K_IN / (gemm_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "nf4_gemm_sm100_pair_kernel<backward> (dX = dY . deq(W), M=4096)",
                "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"], "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                "peak_source": f"{peaks['source']} (cuBLAS bf16 burst)", "ms_per_launch": gemm_ms,
                "traffic": GEMM_BWD_DRAM_BYTES_PER_LAUNCH if m == 4096 else None, "traffic_unit": "bytes per launch (ncu)"}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": m, "n": N_OUT, "k": K_IN, "rank": RANK,
                   "parallelism": f"dp{world}", "l2": "per-step working set (X, dY, Y, dX = 300 MB) exceeds the 126 MB L2",
                   "allreduce": "LoRA gradients (1.18 MB) all-reduced every step on a side stream, overlapping the next step"},
        "frac_of_bf16_peak": value / world / peaks["bf16_tflops"],
        "frac_of_bf16_sustained_peak": value / world / peaks["bf16_tflops_sustained"],
        "sustained": sustained,
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
    }
    del x, dy, y, dx, ws

    extra = {}
    if rank == 0 and world == 1 and not args.no_extras:
        extra = extras(lib, device, desc, packed, state, lora_a, lora_b, peaks)
        check_status("the secondary measurements")
    if not args.no_extras:
        # the metric's second half, at every N: a full QLoRA step at BASELINE config 4's shapes
        torch.cuda.empty_cache()
        from molt_b200.qlora_step import QWEN25_1P5B

        step_line = measure_step(QWEN25_1P5B, "step4", steps=max(3, min(args.steps, 8)), warmup=3, layers=None,
                                 use_graph=True, world=world, rank=rank, local_rank=local_rank, device=device)
        extra["qlora_step_c4"] = {
            "targets_per_s": step_line["value"], "ms_per_step": step_line["ms_per_step"], "n_gpus": world,
            "hot_path_tflops_per_gpu": step_line["hot_path_tflops_per_gpu"],
            "hot_path_frac_of_bf16_peak": step_line["hot_path_frac_of_bf16_peak"],
            "lora_allreduce_bytes": step_line["config"]["lora_parameters"] * 4, "loss": step_line["loss"],
            "gpu_launches": step_line["gpu_launches"], "workload": step_line["config"]["workload"],
            "allreduce": step_line["config"]["allreduce"], "clocks": step_line["clocks"],
        }
    if extra:
        line["extra"] = extra
    if rank == 0 and world == 1:
        base = time_cpu_reference(M_PER_GPU, steps=5, warmup=1)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["cpu_baseline"]["config1"] = time_cpu_config1()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


def profile_case(which, lib, device, desc, packed, state, lora_a, lora_b, x, dy, y, dx, ws, ws_bytes) -> int:
    """Runs one kernel family a few times and exits: the small case an ncu capture is pointed at."""
    from molt_b200 import _native
    from molt_b200.kernels.gated_activation import swiglu_backward, swiglu_forward
    from molt_b200.methods import QuantState, resolved_nf4_scales
    from molt_b200.methods._linear import weight_desc

    stream = _native.stream_handle(device)
    m = x.shape[0]
    plain = QuantState(absmax=resolved_nf4_scales(state), shape=(N_OUT, K_IN), nibble_order=state.nibble_order)
    plain_desc = weight_desc(packed, plain)
    for _ in range(4):
        if which == "gemm_bwd":
            _native.check(lib.molt_nf4_dx(ctypes.byref(plain_desc), dy.data_ptr(), None, None, 0, 0.0, 0, dx.data_ptr(), m,
                                          ws.data_ptr(), ws_bytes, _native.PATH_TCGEN05, stream))
        elif which == "linear_fwd":
            _native.check(lib.molt_nf4_lora_fwd(ctypes.byref(plain_desc), x.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
                                                SCALING, RANK, y.data_ptr(), m, None, ws.data_ptr(), ws_bytes,
                                                _native.PATH_TCGEN05, stream))
        elif which in ("gemv", "gemv1"):
            tokens = 16 if which == "gemv" else 1
            for d in (desc, plain_desc):   # nested absmax (the configuration's own form), then plain fp32 absmax
                _native.check(lib.molt_nf4_gemv(ctypes.byref(d), x.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
                                                SCALING, RANK, y.data_ptr(), tokens, ws.data_ptr(), ws_bytes, stream))
        elif which == "few_tokens":
            for tokens in (16, 64):   # nested absmax, read by the kernel itself
                _native.check(lib.molt_nf4_lora_fwd(ctypes.byref(desc), x.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
                                                    SCALING, RANK, y.data_ptr(), tokens, None, ws.data_ptr(), ws_bytes,
                                                    _native.PATH_FEW_TOKENS, stream))
        elif which == "swiglu":
            gate, up, grad = dy, torch.roll(dy, 1, 0), torch.roll(dy, 2, 0)   # three distinct [M, N] tensors
            swiglu_forward(gate, up)
            swiglu_backward(grad, gate, up)
        else:
            raise SystemExit(f"unknown profile case {which}")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": which, "status": _native.read_status(device)}))
    return 0


def measure_step(shape, workload_name, steps, warmup, layers, use_graph, world, rank, local_rank, device):
    """Times a full QLoRA step of a synthetic-weight decoder (the process group, if any, is already up).
    Returns the JSON line of the step workload as a dict."""
    import torch.distributed as dist

    from molt_b200 import _native
    from molt_b200.qlora_step import QLoRAStep, hot_path_flops_per_token

    lib = _native.library()
    step = QLoRAStep(shape, device, layers=layers, cuda_graph=use_graph, status_interval=0)
    gen = torch.Generator(device=device).manual_seed(1337 + rank)
    tokens = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device=device, generator=gen)
    targets = torch.randint(0, shape.vocab, (shape.micro_batch, shape.seq_len), device=device, generator=gen)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(max(warmup, 3)):
            step.run(tokens, targets)
        barrier()
        launches_before = lib.molt_launch_count() + step.replayed_launches   # eager launches + graph-replayed ones
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as sampler:
            barrier()
            start.record()
            for _ in range(steps):
                loss = step.run(tokens, targets)
            stop.record()
            barrier()
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed.item()) / steps
    step.check_status()
    peaks = measured_peaks()
    n_layers = len(step.model.layers)
    targets_per_s = world * shape.tokens / (ms_per_step * 1e-3)
    hot_flops = hot_path_flops_per_token(shape) * n_layers / shape.layers
    line = {
        "metric": "qlora_step_targets_per_s", "value": targets_per_s, "unit": "targets/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"QLoRA step, {'Qwen2.5-1.5B' if workload_name == 'step4' else 'Llama-3-8B'} architecture, "
                               f"{n_layers} layers, random-init NF4 weights, LoRA r={shape.rank}, seq {shape.seq_len}, "
                               f"micro-batch {shape.micro_batch} per GPU", "parallelism": f"dp{world}",
                   "lora_parameters": step.lora_parameter_count(), "cuda_graph": use_graph,
                   "allreduce": "one bucket per decoder layer, issued from the backward on a side stream, NCCL sum"},
        "hot_path_tflops_per_gpu": hot_flops * shape.tokens / (ms_per_step * 1e-3) / 1e12,
        "hot_path_frac_of_bf16_peak": hot_flops * shape.tokens / (ms_per_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "loss": float(loss), "gpu_launches": int(lib.molt_launch_count() + step.replayed_launches - launches_before),
        "clocks": sampler.summary(),
    }
    del step
    torch.cuda.empty_cache()
    return line


def run_step_workload(args) -> int:
    """BASELINE configs 4 / 5: a full QLoRA step of a synthetic-weight decoder; metric = training targets per second."""
    import torch.distributed as dist

    from molt_b200.qlora_step import LLAMA3_8B, QWEN25_1P5B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")   # keeps NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
    shape = QWEN25_1P5B if args.workload == "step4" else LLAMA3_8B
    line = measure_step(shape, args.workload, args.steps, args.warmup, args.layers, not args.no_graph, world, rank,
                        local_rank, device)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


def extras(lib, device, desc, packed, state, lora_a, lora_b, peaks):
    """Secondary measurements: BASELINE config 2's forward M-sweep, SwiGLU bandwidth, config 3's MLP block."""
    from molt_b200 import _native
    from molt_b200.kernels.gated_activation import swiglu_backward, swiglu_forward
    from molt_b200.methods import QuantState
    from molt_b200.methods._linear import weight_desc
    from molt_b200.modules import GatedMLP, NF4LoRALinear

    out = {}
    gen = torch.Generator(device=device).manual_seed(99)
    sweep = []
    nblocks = N_OUT * K_IN // 64
    # Rotate over copies of the packed weight so that consecutive calls do not find it in the 126 MB L2.
    copies = []
    for _ in range(6):
        st = QuantState(absmax=state.absmax.clone(), shape=state.shape, nested=True, nibble_order=state.nibble_order,
                        state2=state.state2, offset=state.offset)
        pk = packed.clone()
        copies.append((pk, st, weight_desc(pk, st)))
    for m in (1, 8, 16, 32, 64, 128, 256, 1024, 4096, 16384):
        x = torch.randn(m, K_IN, device=device, generator=gen).bfloat16()
        y = torch.empty(m, N_OUT, device=device, dtype=torch.bfloat16)
        ws_bytes = lib.molt_workspace_bytes(_native.OP_LORA_FWD, m, N_OUT, K_IN, RANK)
        ws = torch.empty(ws_bytes, device=device, dtype=torch.uint8)

        def call(d):
            def fn():
                _native.check(lib.molt_nf4_lora_fwd(ctypes.byref(d), x.data_ptr(), lora_a.data_ptr(), lora_b.data_ptr(),
                                                    SCALING, RANK, y.data_ptr(), m, None, ws.data_ptr(), ws_bytes,
                                                    _native.PATH_AUTO, _native.stream_handle(device)))
            return fn

        ms = graph_time_ms([call(c[2]) for c in copies], replays=20 if m <= 1024 else 3)
        flops = linear_flops(m, backward=False)
        bytes_alg = N_OUT * K_IN // 2 + nblocks + nblocks // 256 * 4 + m * K_IN * 2 + m * N_OUT * 2 + RANK * (K_IN + N_OUT) * 4
        sweep.append({"m": m, "ms": ms, "path": "gemv" if m <= 8 else "few_tokens" if m <= 128 else "tcgen05", "tflops": flops / ms / 1e9,
                      "frac_bf16_peak": flops / ms / 1e9 / peaks["bf16_tflops"],
                      "gbs": bytes_alg / ms / 1e6, "frac_hbm": bytes_alg / ms / 1e6 / peaks["hbm_gbs"]})
    del copies
    out["forward_sweep_config2"] = sweep

    # per-shape table of the projections of BASELINE configs 3 / 4 at 8192 tokens: forward linear (low-rank term and
    # side kernels included) and the input-gradient GEMM alone
    shapes = []
    for n, k in ((8960, 1536), (1536, 8960), (1536, 1536), (256, 1536)):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        from molt_b200.methods import quantize_nf4
        pk, st = quantize_nf4(w, 64, False)
        d = weight_desc(pk, st)
        a = torch.randn(RANK, k, device=device, generator=gen) * 0.01
        b = torch.randn(n, RANK, device=device, generator=gen) * 0.01
        m = 8192
        x = torch.randn(m, k, device=device, generator=gen).bfloat16()
        dy = torch.randn(m, n, device=device, generator=gen).bfloat16()
        y = torch.empty(m, n, device=device, dtype=torch.bfloat16)
        dx = torch.empty(m, k, device=device, dtype=torch.bfloat16)
        ws_bytes = max(lib.molt_workspace_bytes(_native.OP_LORA_FWD, m, n, k, RANK), lib.molt_workspace_bytes(_native.OP_DX, m, n, k, RANK))
        ws = torch.empty(ws_bytes, device=device, dtype=torch.uint8)
        stream = _native.stream_handle(device)
        fwd_ms = event_time_ms(lambda: _native.check(lib.molt_nf4_lora_fwd(
            ctypes.byref(d), x.data_ptr(), a.data_ptr(), b.data_ptr(), SCALING, RANK, y.data_ptr(), m, None, ws.data_ptr(),
            ws_bytes, _native.PATH_AUTO, stream)), iters=10, warmup=3)
        dx_ms = event_time_ms(lambda: _native.check(lib.molt_nf4_dx(
            ctypes.byref(d), dy.data_ptr(), None, None, 0, 0.0, 0, dx.data_ptr(), m, ws.data_ptr(), ws_bytes,
            _native.PATH_AUTO, stream)), iters=10, warmup=3)
        flops = 2.0 * m * n * k
        shapes.append({"n": n, "k": k, "m": m, "forward_ms": fwd_ms, "forward_frac_bf16_peak": flops / fwd_ms / 1e9 / peaks["bf16_tflops"],
                       "dx_gemm_ms": dx_ms, "dx_gemm_frac_bf16_peak": flops / dx_ms / 1e9 / peaks["bf16_tflops"]})
        del w, pk, x, dy, y, dx, ws
    out["projection_shapes_config3_4"] = shapes

    rows, inter, hidden = 8192, 8960, 1536
    g = torch.randn(rows, inter, device=device, generator=gen).bfloat16()
    u = torch.randn(rows, inter, device=device, generator=gen).bfloat16()
    d = torch.randn(rows, inter, device=device, generator=gen).bfloat16()
    count = rows * inter
    fwd_ms = event_time_ms(lambda: swiglu_forward(g, u), iters=10, warmup=3)
    bwd_ms = event_time_ms(lambda: swiglu_backward(d, g, u), iters=10, warmup=3)
    out["swiglu_config3"] = {
        "elements": count,
        "fwd": {"ms": fwd_ms, "gbs": 6 * count / fwd_ms / 1e6, "frac_hbm": 6 * count / fwd_ms / 1e6 / peaks["hbm_gbs"]},
        "bwd": {"ms": bwd_ms, "gbs": 10 * count / bwd_ms / 1e6, "frac_hbm": 10 * count / bwd_ms / 1e6 / peaks["hbm_gbs"]},
    }
    del g, u, d

    def proj(n, k):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        lin = NF4LoRALinear.from_dense(w, RANK, ALPHA, nibble_order="low-first")
        with torch.no_grad():
            lin.lora_B["default"].weight.normal_(0, 0.01, generator=gen)
        return lin

    mlp = GatedMLP(proj(inter, hidden), proj(inter, hidden), proj(hidden, inter))
    x = torch.randn(rows, hidden, device=device, generator=gen).bfloat16()
    dy = torch.randn(rows, hidden, device=device, generator=gen).bfloat16()

    def block_step():
        xin = x.detach().requires_grad_()
        mlp.fused(xin, rematerialize_up=True).backward(dy)

    eager_ms = event_time_ms(block_step, iters=5, warmup=2)   # through Python autograd: includes host launch gaps
    # the same step replayed as a CUDA graph, as the step driver (and the reference's trainer) runs it: device time
    ms = graph_time_ms([block_step], replays=10)
    flops = 3 * linear_flops(rows, inter, hidden)
    out["mlp_block_config3"] = {"ms": ms, "tflops_algorithmic": flops / ms / 1e9,
                                "frac_bf16_peak": flops / ms / 1e9 / peaks["bf16_tflops"], "replay_up": True,
                                "timing": "one forward+backward of the block captured as a CUDA graph, replayed 10 times",
                                "ms_eager_autograd": eager_ms}
    return out


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-extras", action="store_true", help="skip the secondary measurements")
    parser.add_argument("--workload", choices=("linear", "step4", "step5"), default="linear",
                        help="linear = the headline NF4-LoRA linear; step4 / step5 = full QLoRA step of BASELINE config 4 / 5")
    parser.add_argument("--no-graph", action="store_true", help="step workloads: run eagerly instead of replaying a CUDA graph")
    parser.add_argument("--layers", type=int, default=None, help="step workloads: use fewer decoder layers")
    parser.add_argument("--profile", choices=("gemm_bwd", "linear_fwd", "gemv", "gemv1", "few_tokens", "swiglu"), default=None,
                        help="run one kernel family four times and exit (target of an ncu capture)")
    args = parser.parse_args()
    if args.steps < 1:
        parser.error("--steps must be positive")
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload != "linear":
        return run_step_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
