#!/usr/bin/env python
"""Benchmark of the O0/O1/O2 quantized-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload (N = 1): the canonical experiment M = N = K = 4096 with seeded synthetic inputs of the
canonical distributions.  One *step* is one steady-state pass of all three variants on one batch of
activations: O0 (INT8->FP16 conversion + FP16 GEMM), O1 (INT8 GEMM with per-K32 FP32 rescale) and
O2 (MXFP4 re-quantization + block-scaled MXFP4 GEMM); the weight-side conversions are cached, as in
the reference's ``steady_state`` mode.  The metric is equivalent TFLOP/s, ``2*M*N*K`` per variant
per step divided by time.  With N GPUs, W is sharded along its rows (global N = 4096 * N_gpus,
4096 per GPU), A is broadcast once before timing, and no collective is on the timed path.

The JSON line also carries: per-kernel timings and roofline fractions measured with CUDA events
inside the timed steps, an end-to-end figure through the host-buffer C ABI (pinned host A in,
Y back to the host), sampled GPU clocks, and a CPU baseline (the numpy oracle on a bounded sample
of the same workload, on this machine's cores).

``--impl reference`` times the reference's CPU algorithm (the oracle port) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N_PER_GPU = K = 4096
VARIANTS = ("o0", "o1", "o2")
FLOP_PER_VARIANT = 2.0 * M * N_PER_GPU * K
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch at 4096^3 from an ncu capture of one
# benchmark step (summary kept under profiles/; the 126 MB L2 keeps most of the 64 MiB output on chip)
NCU_DRAM_TRAFFIC_BYTES = {"o0_int8_to_fp16": 16.8e6, "o0_gemm_f16": 124.7e6, "o1_int8_to_bf16": 16.8e6,
                          "o1_gemm_bf16": 114.9e6, "o1_gemm_i8": 52.1e6, "o2_quantize": 16.8e6, "o2_gemm_mxf4": 32.4e6}
# every INT32 K32 partial of O1 is converted, multiplied and accumulated in FP32 by the epilogue warps:
# 3 issue cycles per partial per warp (measured in isolation with four warps per scheduler), 4 schedulers per SM
O1_ISSUE_CYCLES_PER_PARTIAL = 3.0
# with BF16 operands (weight scale folded into W) the partial arrives as an exact FP32 product: multiply + add
O1_BF16_ISSUE_CYCLES_PER_PARTIAL = 2.0


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- clock sampling -------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# ---- CPU baseline / reference arm -----------------------------------------------------------------------

def cpu_sample_inputs(rows: int):
    """The first `rows` activations of the canonical 4096^3 sample and the full weights (numpy)."""
    from adangel_oyzl_b200 import synthetic

    p = synthetic.canonical_inputs(M, N_PER_GPU, K)
    return (p.A_int8[:rows].numpy().copy(), p.A_scale[:rows].numpy().copy(), p.W_mxfp4.numpy(), p.W_scale.numpy())


def time_cpu_oracle(rows: int, steps: int, warmup: int):
    """Seconds per steady-state step of the oracle on a `rows`-row sample (weights prepared once)."""
    from oracle import adangel_oracle as orc

    a_int8, a_scale, w_mx, w_sc = cpu_sample_inputs(rows)
    prepared = orc.prepare_weights(w_mx, w_sc)
    for _ in range(warmup):
        orc.steady_state_step(a_int8, a_scale, prepared)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.steady_state_step(a_int8, a_scale, prepared)
    return (time.perf_counter() - t0) / steps


def cpu_baseline_record(rows: int, seconds_per_step: float) -> dict:
    flops = len(VARIANTS) * 2.0 * rows * N_PER_GPU * K
    return {
        "value": flops / seconds_per_step / 1e12,
        "unit": "TFLOP/s",
        "cores": os.cpu_count(),
        "kind": "port",
        "sample": f"numpy oracle, steady-state O0+O1+O2 on the first {rows} of 4096 activation rows x full 4096x4096 W "
                  f"(rows are independent; weights prepared once), {seconds_per_step:.3f} s/step",
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 256
    sec = time_cpu_oracle(rows, args.steps, args.warmup)
    base = cpu_baseline_record(rows, sec)
    line = {
        "impl": "reference",
        "metric": "O0+O1+O2 steady-state equivalent TFLOP/s at 4096^3 (2*M*N*K per variant)",
        "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (CPU: fp32 matmul of integer-valued / dequantized operands)", "data": "synthetic",
        "config": {"workload": "canonical 4096^3 O0+O1+O2 steady state, CPU sample of 256 activation rows"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- native arm ------------------------------------------------------------------------------------------

def run_native_arm(args) -> None:
    import torch

    from adangel_oyzl_b200 import kernels, parallel, synthetic
    from adangel_oyzl_b200.ops.extension import require_native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    require_native()  # fails loudly when the CUDA library is missing or the GPU is not a B200
    peaks = measured_peaks()

    # inputs: global problem M x (4096 * world) x K; this rank owns rows [rank*4096, (rank+1)*4096) of W
    n_global = N_PER_GPU * world
    a_f, _ = synthetic.canonical_floats(M, 1, K)
    if rank == 0:
        a_int8, a_scale = synthetic.quantize_int8_per_row(a_f.to(dev))
    else:
        a_int8 = torch.empty((M, K), dtype=torch.int8, device=dev)
        a_scale = torch.empty((M,), dtype=torch.float32, device=dev)
    if distributed:
        parallel.broadcast_activations(a_int8, a_scale, src=0)
    g = torch.Generator().manual_seed(synthetic.CANONICAL_SEED + 1 + rank)
    w_f = torch.randn(N_PER_GPU, K, generator=g, dtype=torch.float32) * 0.02
    w_mxfp4, w_scale = synthetic.quantize_mxfp4(w_f.to(dev))
    n0, n1 = parallel.shard_range(n_global, world, rank)
    assert n1 - n0 == N_PER_GPU
    shard = parallel.ShardedWeights(n0, n1, w_mxfp4, w_scale)
    shard.w_fp16 = kernels.mxfp4_to_fp16(w_mxfp4, w_scale)
    shard.w_int8 = kernels.mxfp4_to_int8(w_mxfp4)
    # O1 runs on BF16 operands (weight scale folded into W; bit-identical to the INT8-operand kernel) when
    # the operands lie inside that kernel's exact range, which the conversions report in `o1_flag`
    o1_flag = kernels.new_range_flag(dev)
    shard.w_bf16 = kernels.mxfp4_to_bf16_scaled(w_mxfp4, w_scale, o1_flag)
    a_bf16 = kernels.int8_to_bf16(a_int8, a_scale, o1_flag)
    o1_on_bf16 = int(o1_flag.item()) == 0
    shard.w_sf_tiled = kernels.o2_tile_scales(w_scale)

    # per-variant buffers (distinct outputs so a step's working set exceeds L2)
    y = {v: torch.empty((M, N_PER_GPU), dtype=torch.float32, device=dev) for v in VARIANTS}
    lib = kernels._lib()
    stream = torch.cuda.current_stream(dev)
    sp = stream.cuda_stream
    a16 = torch.empty((M, K), dtype=torch.float16, device=dev)
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    sfa = torch.zeros((kernels.tiled_scale_bytes(M, K),), dtype=torch.uint8, device=dev)
    check = kernels._sm100._check

    o1_gemm_name = "o1_gemm_bf16" if o1_on_bf16 else "o1_gemm_i8"
    kernel_names = ("o0_int8_to_fp16", "o0_gemm_f16", "o1_int8_to_bf16", o1_gemm_name, "o2_quantize", "o2_gemm_mxf4")

    def o1_int8_gemm():
        check(lib.adg_gemm_o1(a_int8.data_ptr(), a_scale.data_ptr(), shard.w_int8.data_ptr(), shard.w_scale.data_ptr(),
                              y["o1"].data_ptr(), None, M, N_PER_GPU, K, N_PER_GPU, sp))

    def step(events=None):
        def mark(i):
            if events is not None:
                events[i].record(stream)
        mark(0)
        check(lib.adg_int8_to_fp16(a_int8.data_ptr(), a_scale.data_ptr(), a16.data_ptr(), M, K, sp))
        mark(1)
        check(lib.adg_gemm_o0(a16.data_ptr(), shard.w_fp16.data_ptr(), y["o0"].data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))
        mark(2)
        if o1_on_bf16:
            check(lib.adg_int8_to_bf16(a_int8.data_ptr(), a_scale.data_ptr(), a_bf16.data_ptr(), o1_flag.data_ptr(), M, K, sp))
            mark(3)
            check(lib.adg_gemm_o1_bf16(a_bf16.data_ptr(), a_scale.data_ptr(), shard.w_bf16.data_ptr(), y["o1"].data_ptr(),
                                       o1_flag.data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))
        else:
            mark(3)
            o1_int8_gemm()
        mark(4)
        check(lib.adg_o2_quantize_activation(a_int8.data_ptr(), a_scale.data_ptr(), codes.data_ptr(), None,
                                             sfa.data_ptr(), M, K, sp))
        mark(5)
        check(lib.adg_gemm_o2(codes.data_ptr(), sfa.data_ptr(), shard.w_mxfp4.data_ptr(), shard.w_sf_tiled.data_ptr(),
                              y["o2"].data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))
        mark(6)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    kernels.check_status(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # timed region: exactly `steps` steps between two events, barrier + synchronize on both sides
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record(stream)
    for _ in range(args.steps):
        step()
    t_end.record(stream)
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    # breakdown pass: the same steps again with an event between consecutive kernels
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps)]
    for i in range(args.steps):
        step(events[i])
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    kernels.check_status(dev)
    if distributed:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * len(VARIANTS) * FLOP_PER_VARIANT / (ms_per_step * 1e-3) / 1e12

    # conversion kernels are a few microseconds long: also time them as the reference's protocol
    # does, as batches of back-to-back launches, rotating over buffers so that L2 does not serve them
    def batched(fn, reps=50):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn(0)
        e0.record(stream)
        for i in range(reps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps

    n_rot = 6  # 6 x (16 MiB in + 32 MiB out) > L2
    a_rot = [a_int8.clone() for _ in range(n_rot)]
    a16_rot = [torch.empty_like(a16) for _ in range(n_rot)]
    abf_rot = [torch.empty_like(a_bf16) for _ in range(n_rot)]
    codes_rot = [torch.empty_like(codes) for _ in range(n_rot)]
    batched_ms = {
        "o0_int8_to_fp16": batched(lambda i: check(lib.adg_int8_to_fp16(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), a16_rot[i % n_rot].data_ptr(), M, K, sp))),
        "o1_int8_to_bf16": batched(lambda i: check(lib.adg_int8_to_bf16(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), abf_rot[i % n_rot].data_ptr(), o1_flag.data_ptr(), M, K, sp))),
        "o2_quantize": batched(lambda i: check(lib.adg_o2_quantize_activation(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), codes_rot[i % n_rot].data_ptr(), None, sfa.data_ptr(), M, K, sp))),
    }
    del a_rot, a16_rot, abf_rot, codes_rot
    # the INT8-operand O1 kernel, for comparison (outside the timed region; same bits in y["o1"])
    y1_bf16 = y["o1"].clone()
    o1_int8_ms = batched(lambda i: o1_int8_gemm(), reps=10)
    o1_same_bits = bool(torch.equal(y1_bf16, y["o1"]))
    del y1_bf16

    # per-kernel durations from the events recorded inside the timed steps
    kernel_ms = {name: statistics.fmean(events[i][j].elapsed_time(events[i][j + 1]) for i in range(args.steps))
                 for j, name in enumerate(kernel_names)}
    mse = {v: float(((y[v].double() - y["o0"].double()) ** 2).mean()) for v in ("o1", "o2")}

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    conv_bytes = {"o0_int8_to_fp16": M * K + 4 * M + 2 * M * K, "o1_int8_to_bf16": M * K + 4 * M + 2 * M * K,
                  "o2_quantize": M * K + 4 * M + M * K // 2 + M * K // 32}
    # tensor peak per kernel: the measured BF16 cuBLAS burst times the MMA kind's nominal ratio to BF16
    peak_mult = {"o0_gemm_f16": 1.0, "o1_gemm_bf16": 1.0, "o1_gemm_i8": 2.0, "o2_gemm_mxf4": 4.0}
    nominal = {"o0_gemm_f16": 2250.0, "o1_gemm_bf16": 2250.0, "o1_gemm_i8": 4500.0, "o2_gemm_mxf4": 9000.0}
    kernels_out = {}
    if o1_on_bf16:
        kernel_ms = dict(kernel_ms, o1_gemm_i8=o1_int8_ms)
    else:
        kernel_ms.pop("o1_int8_to_bf16")
        batched_ms.pop("o1_int8_to_bf16")
    for name, ms in kernel_ms.items():
        if name in conv_bytes:
            ach = conv_bytes[name] / (ms * 1e-3) / 1e9
            bms = batched_ms[name]
            bach = conv_bytes[name] / (bms * 1e-3) / 1e9
            kernels_out[name] = {"ms": ms, "bound": "hbm", "achieved": ach, "unit": "GB/s", "peak": peaks["hbm_gbs"],
                                 "frac": ach / peaks["hbm_gbs"], "algorithmic_bytes": conv_bytes[name],
                                 "batched_ms": bms, "batched_achieved": bach, "batched_frac": bach / peaks["hbm_gbs"]}
        else:
            ach = FLOP_PER_VARIANT / (ms * 1e-3) / 1e12
            peak = peaks["bf16_tflops"] * peak_mult[name]
            kernels_out[name] = {"ms": ms, "bound": "tensor", "achieved": ach, "unit": "TFLOP/s", "peak": peak,
                                 "frac": ach / peak, "frac_of_nominal": ach / nominal[name]}
    if o1_on_bf16:
        kernels_out["o1_gemm_i8"]["note"] = ("INT8-operand O1 kernel, timed outside the step for comparison; "
                                             f"bit-identical output: {o1_same_bits}")
    dominant = max((k for k in kernel_ms if not (o1_on_bf16 and k == "o1_gemm_i8")), key=kernel_ms.get)
    d = kernels_out[dominant]
    roofline = {"kernel": dominant, "bound": d["bound"], "achieved": d["achieved"], "peak": d["peak"], "unit": d["unit"],
                "frac": d["frac"], "traffic": NCU_DRAM_TRAFFIC_BYTES.get(dominant),
                "peak_source": f"{peaks['source']}: bf16 cuBLAS burst x{peak_mult[dominant]:g}" if d["bound"] == "tensor"
                else f"{peaks['source']}: HBM copy"}

    if dominant in ("o1_gemm_i8", "o1_gemm_bf16") and clocks and clocks.get("sm_mhz"):
        partials = M * N_PER_GPU * (K // 32)
        cycles = O1_ISSUE_CYCLES_PER_PARTIAL if dominant == "o1_gemm_i8" else O1_BF16_ISSUE_CYCLES_PER_PARTIAL
        floor_s = partials * cycles / 32 / (148 * 4 * clocks["sm_mhz"] * 1e6)
        roofline["secondary_bound"] = {
            "what": "FP32 issue slots of the epilogue: every K32 partial is scaled and accumulated separately (literal O1 "
                    f"semantics: one rounding per step and operation), {cycles:g} issue cycles per partial per warp",
            "floor_ms": floor_s * 1e3, "frac_of_floor": floor_s * 1e3 / d["ms"]}

    # end to end through the host-buffer C ABI (N = 1 only): pinned A in, Y back, every variant, every step
    e2e = None
    if not distributed:
        a_host = torch.empty((M, K), dtype=torch.int8).pin_memory()
        s_host = torch.empty((M,), dtype=torch.float32).pin_memory()
        a_host.copy_(a_int8.cpu())
        s_host.copy_(a_scale.cpu())
        y_host = {v: torch.empty((M, N_PER_GPU), dtype=torch.float32).pin_memory() for v in VARIANTS}
        w_mx_host, w_sc_host = w_mxfp4.cpu().contiguous(), w_scale.cpu().contiguous()
        sessions = {v: kernels.HostSession(v, M, w_mx_host, w_sc_host) for v in VARIANTS}
        e2e_steps = max(3, min(args.steps, 10))

        def e2e_step():
            # the three variants' passes are submitted back to back (each on its session's stream), so
            # one variant's copies overlap another's kernels; the step ends when every Y is in host memory
            for v in VARIANTS:
                sessions[v].submit(a_host, s_host, y_host[v])
            for v in VARIANTS:
                sessions[v].wait()

        e2e_step()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_sec = (time.perf_counter() - t0) / e2e_steps
        for s in sessions.values():
            s.close()
        e2e = {"value": len(VARIANTS) * FLOP_PER_VARIANT / e2e_sec / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": len(VARIANTS) * (M * K + 4 * M), "d2h_bytes_per_step": len(VARIANTS) * 4 * M * N_PER_GPU,
               "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps,
               "path": "adg_session_submit/wait (C ABI, pinned host buffers): H2D A + conversion + GEMM + D2H Y per variant, "
                       "the three variants' passes in flight together"}

    cpu = None
    if not distributed and not args.no_cpu_baseline:
        rows = 512
        cpu = cpu_baseline_record(rows, time_cpu_oracle(rows, 3, 1))

    working_set = (M * K + 2 * M * K + 2 * M * K + M * K // 2) + (2 + 2 + 0.5) * N_PER_GPU * K + 3 * 4 * M * N_PER_GPU
    line = {
        "metric": "O0+O1+O2 steady-state equivalent TFLOP/s at 4096^3 (2*M*N*K per variant)",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 / bf16 (exact integers, O1) / mxf4 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"canonical M=4096 K=4096, N=4096 per GPU (W sharded by rows, global N={n_global}), "
                               "steady state: activation conversion + GEMM for O0, O1 and O2",
                   "l2": f"no flush: each step touches about {working_set / 2**20:.0f} MiB > 126 MiB L2",
                   "seed": synthetic.CANONICAL_SEED},
        "variants": {
            "o0": {"gemm_tflops": kernels_out["o0_gemm_f16"]["achieved"],
                   "steady_tflops": FLOP_PER_VARIANT / ((kernel_ms["o0_int8_to_fp16"] + kernel_ms["o0_gemm_f16"]) * 1e-3) / 1e12},
            "o1": {"gemm_tflops": kernels_out[o1_gemm_name]["achieved"],
                   "steady_tflops": FLOP_PER_VARIANT / ((kernel_ms.get("o1_int8_to_bf16", 0.0) + kernel_ms[o1_gemm_name]) * 1e-3) / 1e12,
                   "operands": "bf16 (weight scale folded into W)" if o1_on_bf16 else "int8"},
            "o2": {"gemm_tflops": kernels_out["o2_gemm_mxf4"]["achieved"],
                   "steady_tflops": FLOP_PER_VARIANT / ((kernel_ms["o2_quantize"] + kernel_ms["o2_gemm_mxf4"]) * 1e-3) / 1e12},
        },
        "mse_vs_o0": mse,
        "kernels": kernels_out,
        "roofline": roofline,
        "clocks": clocks,
        "e2e": e2e,
        "cpu_baseline": cpu,
        "gpu_launches": (6 if o1_on_bf16 else 5) * args.steps,
        "timing": "value: two CUDA events around all steps; kernels: a second pass with an event between kernels "
                  "(adds about a microsecond per boundary); batched_*: 50 back-to-back launches over rotating buffers",
    }
    print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("native", "reference"), default="native")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle timing in the native arm")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_native_arm(args)


if __name__ == "__main__":
    main()
