#!/usr/bin/env python
"""Benchmark of the O0/O1/O2 quantized-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload (N = 1): the canonical experiment M = N = K = 4096 with seeded synthetic inputs of the canonical
distributions.  One *pass* is the steady state of all three variants on one batch of activations: O0 (INT8 ->
FP16 conversion + FP16 GEMM), O1 (INT8 -> BF16 conversion + the per-K32 recurrence on BF16 operands,
bit-identical to the INT8-operand kernel) and O2 (MXFP4 re-quantization + block-scaled GEMM): six kernels; the
weight-side conversions are cached, as in the reference's ``steady_state`` mode.  One *step* is
``passes_per_step`` passes, sized so that the K timed steps last at least two seconds: the sampled SM clocks
and power then belong to the kernels, and ``value`` is a sustained figure.  The metric is equivalent TFLOP/s,
``2*M*N*K`` per variant and pass.  A short burst of K passes is timed as well (``config.burst``).  With N GPUs,
W is sharded along its rows (global N = 4096 * N_gpus, 4096 per GPU), A is broadcast once before timing, and no
collective is on the timed path; in addition every run measures the N-sharded 16384 x 28672 x 8192 problem
(strong scaling: total work fixed) for O1 and O2 and reports it in ``config.sharded_16384x28672x8192``.

The JSON line also carries per-kernel timings and roofline fractions measured with CUDA events, an end-to-end
figure through the host-buffer C ABI (pinned host A in, Y back to the host), sampled GPU clocks, and a CPU
baseline: the reference project's own Python path (``oracle/_ref``, see ``oracle/make_ref.py``) on a bounded
row sample of the same workload on this machine's cores, or the numpy oracle port where that copy is absent.

``--impl reference`` times that CPU path alone.
"""

from __future__ import annotations

import argparse
import json
import os
import re
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
SHARDED = (16384, 28672, 8192)
MIN_TIMED_SECONDS = 2.0
CPU_SAMPLE_ROWS = 256
# every K32 partial of O1 is multiplied by the activation scale and accumulated in FP32 by the epilogue warps:
# with BF16 operands (weight scale folded into W) that is two issue cycles per partial and warp, three with INT8 operands
O1_ISSUE_CYCLES = {"o1_gemm_bf16": 2.0, "o1_gemm_i8": 3.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_dram_traffic() -> dict:
    """DRAM bytes per launch (read + write) of the step's kernels, from the committed ncu summary
    ``profiles/bench_step_kernels_full_4096.md`` (the rows ``dram__bytes_read.sum`` / ``dram__bytes_write.sum``
    of its table, in MB, one column per kernel)."""
    path = ROOT / "profiles" / "bench_step_kernels_full_4096.md"
    if not path.exists():
        return {}
    header, rows = None, {}
    for line in path.read_text(encoding="utf-8").splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if line.startswith("| metric"):
            header = cells[1:]
        elif header and line.startswith("| dram__bytes_"):
            rows[cells[0].split()[0]] = cells[1:]
    if not header or len(rows) < 2:
        return {}
    out = {}
    for i, name in enumerate(header):
        try:
            total = sum(float(re.match(r"[-+0-9.eE]+", rows[key][i]).group(0)) for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"))
        except (AttributeError, IndexError, KeyError):
            continue
        out[name] = total * 1e6
    return out


# ---- clock sampling -------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks, power and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

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
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, window=None) -> dict:
        """`window` = (t0, t1) in perf_counter time: only samples taken inside it count as "under load"."""
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
        total = 0
        for stamp, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            total += 1
            if window is not None and not (window[0] <= stamp <= window[1]):
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
            "power_w_median": statistics.median(power) if power else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "samples_total": total,
            "reasons": sorted(reasons),
        }


# ---- CPU baseline / reference arm -----------------------------------------------------------------------

def cpu_sample_inputs(rows: int):
    """The first `rows` activations of the canonical 4096^3 sample and the full weights (CPU torch tensors)."""
    from adangel_oyzl_b200 import synthetic

    p = synthetic.canonical_inputs(M, N_PER_GPU, K)
    return p.A_int8[:rows].contiguous(), p.A_scale[:rows].contiguous(), p.W_mxfp4, p.W_scale


def reference_package():
    """The reference project's own Python package from ``oracle/_ref`` (None when the copy is absent)."""
    ref = ROOT / "oracle" / "_ref"
    if not (ref / "adangel" / "reference").is_dir():
        return None
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    try:
        from adangel.reference import run_o0_reference, run_o1_reference, run_o2_reference
        from adangel.trace.schema import PreparedInputs
    except Exception:
        return None
    return {"run": (run_o0_reference, run_o1_reference, run_o2_reference), "inputs": PreparedInputs}


def time_cpu_path(rows: int, steps: int, warmup: int):
    """Seconds per pass of the CPU arm on a `rows`-row sample, and what was timed."""
    import torch

    torch.set_num_threads(os.cpu_count() or 1)
    a_int8, a_scale, w_mx, w_sc = cpu_sample_inputs(rows)
    ref = reference_package()
    if ref is not None:
        inputs = ref["inputs"]("bench_sample", a_int8, a_scale, w_mx, w_sc)

        def one_pass():
            for fn in ref["run"]:
                fn(inputs)
        kind = "reference"
        what = ("the reference's own run_o0_reference + run_o1_reference + run_o2_reference (python/adangel/reference, torch on CPU; "
                "each call includes its own weight-side conversion: the reference has no cached-weight CPU path)")
    else:
        from oracle import adangel_oracle as orc

        args = tuple(t.numpy() for t in (a_int8, a_scale))
        prepared = orc.prepare_weights(w_mx.numpy(), w_sc.numpy())

        def one_pass():
            orc.steady_state_step(args[0], args[1], prepared)
        kind = "port"
        what = "numpy oracle port, steady-state O0+O1+O2 with weights prepared once (oracle/_ref is absent on this machine)"
    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    return (time.perf_counter() - t0) / steps, kind, what


def cpu_baseline_record(rows: int, seconds: float, kind: str, what: str) -> dict:
    flops = len(VARIANTS) * 2.0 * rows * N_PER_GPU * K
    return {
        "value": flops / seconds / 1e12,
        "unit": "TFLOP/s",
        "cores": os.cpu_count(),
        "kind": kind,
        "sample": f"{what}; the first {rows} of 4096 activation rows x the full 4096x4096 W (rows of Y are independent), "
                  f"{seconds:.3f} s per pass",
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sec, kind, what = time_cpu_path(CPU_SAMPLE_ROWS, args.steps, min(args.warmup, 2))
    base = cpu_baseline_record(CPU_SAMPLE_ROWS, sec, kind, what)
    line = {
        "impl": "reference",
        "metric": "O0+O1+O2 steady-state equivalent TFLOP/s at 4096^3 (2*M*N*K per variant)",
        "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 / int32 on CPU (torch)", "data": "synthetic",
        "config": {"workload": f"canonical 4096^3 O0+O1+O2, CPU sample of {CPU_SAMPLE_ROWS} activation rows, one pass per step"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- the N-sharded large shape (strong scaling) -------------------------------------------------------------

def sharded_block(dist, world: int, rank: int, dev) -> dict:
    """16384 x 28672 x 8192 with W split by rows over the ranks, A replicated: steady-state O1 and O2 per rank
    (max over ranks), the stand-alone re-quantization kernel, and the gather of Y's column blocks."""
    import torch

    from adangel_oyzl_b200 import kernels, parallel

    m, n, k = SHARDED
    g = torch.Generator(device=dev).manual_seed(20250805)
    a = torch.randn((m, k), generator=g, device=dev)
    idx = torch.randperm(k, generator=g, device=dev)[: max(1, round(0.005 * k))]
    a[:, idx] *= 20.0
    a_int8, a_scale = kernels.quantize_int8_per_row(a, check_finite=False)
    del a
    if dist is not None:
        parallel.broadcast_activations(a_int8, a_scale, src=0)  # once, outside every timed region
    n0, n1 = parallel.shard_range(n, world, rank)
    g = torch.Generator(device=dev).manual_seed(20250805 + 1000 + rank)
    w = torch.randn((n1 - n0, k), generator=g, device=dev) * 0.02
    w_mxfp4, w_scale = kernels.quantize_mxfp4(w, check_finite=False)
    del w
    shard = parallel.shard_weights(w_mxfp4, w_scale, 1, 0, variants=("o1", "o2"))
    shard.n0, shard.n1 = n0, n1
    y = torch.empty((m, n1 - n0), dtype=torch.float32, device=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, warmup, reps):
        for _ in range(warmup):
            fn()
        kernels.check_status(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / reps)

    flop = 2.0 * m * n * k
    o1_ms = timed(lambda: parallel.sharded_gemm("o1", a_int8, a_scale, shard, out=y), 1, 3)
    o2_ms = timed(lambda: parallel.sharded_gemm("o2", a_int8, a_scale, shard, out=y), 2, 10)
    o2_one_kernel_ms = timed(lambda: parallel.sharded_gemm("o2", a_int8, a_scale, shard, out=y, fused=True), 2, 10)
    o2_quantize_ms = timed(lambda: kernels.o2_quantize_activation(a_int8, a_scale, want_natural=False), 2, 10)
    out = {
        "shape": [m, n, k], "scaling": "strong", "n_gpus": world, "rows_of_w_per_rank": n1 - n0,
        "o1_ms": o1_ms, "o1_aggregate_tflops": flop / o1_ms / 1e9,
        "o2_ms": o2_ms, "aggregate_tflops": flop / o2_ms / 1e9,
        "o2_one_kernel_ms": o2_one_kernel_ms, "o2_quantize_ms": o2_quantize_ms,
        "o1_path": "adg_o1_linear (INT8 -> BF16 conversion + BF16-operand kernel, INT8-operand kernel behind it)",
        "o2_path": "adg_o2_linear (re-quantization of the replicated A, then the GEMM; o2_one_kernel_ms: the GEMM kernel that "
                   "re-quantizes A itself)",
        "timing": "CUDA events around back-to-back calls, barrier + synchronize on both sides, max over ranks",
        "gather_ms": None,
    }
    if dist is not None:
        full = parallel.gather_columns(y, n)  # warm-up (NCCL set-up, allocator)
        del full
        times = []
        for _ in range(3):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            full = parallel.gather_columns(y, n)
            e1.record()
            barrier()
            times.append(max_over_ranks(e0.elapsed_time(e1)))
            if len(times) < 3:
                del full
        out["gather_ms"] = min(times)
        out["gather_ms_all"] = times
        out["gather_received_gb_per_gpu"] = 4.0 * m * (n - (n1 - n0)) / 1e9
        out["gather_tb_per_s_received"] = out["gather_received_gb_per_gpu"] / out["gather_ms"]
        assert tuple(full.shape) == (m, n)
        # the same gather by this rank's own kernel reading the peers' blocks over NVLink (no staging, no permute)
        try:
            peers = parallel.PeerGather(m, n, dev)
        except RuntimeError as exc:  # raised on every rank or on none
            out["gather_peer_ms"] = None
            out["gather_peer_error"] = str(exc)[:200]
            peers = None
        if peers is not None:
            peers.block.copy_(y)
            peers.gather(out=full)  # warm-up
            times = []
            for _ in range(3):
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                peers.gather(out=full)
                e1.record()
                barrier()
                times.append(max_over_ranks(e0.elapsed_time(e1)))
            out["gather_peer_ms"] = min(times)
            out["gather_peer_ms_all"] = times
            out["gather_peer_tb_per_s_received"] = out["gather_received_gb_per_gpu"] / out["gather_peer_ms"]
            out["gather_peer_path"] = ("adg_gather_columns_pull: one kernel per rank, 16-byte loads from the peers' memory (CUDA IPC), "
                                       "a one-element all-reduce before and after it inside the timed region")
            peers.close()
        del full
    kernels.check_status(dev)
    return out


# ---- native arm ------------------------------------------------------------------------------------------

def run_native_arm(args) -> None:
    import torch

    from adangel_oyzl_b200 import kernels, parallel, synthetic
    from adangel_oyzl_b200.ops import _sm100
    from adangel_oyzl_b200.ops.extension import require_native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
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
    w_fp16 = kernels.mxfp4_to_fp16(w_mxfp4, w_scale)
    w_int8 = kernels.mxfp4_to_int8(w_mxfp4)
    # O1 runs on BF16 operands (weight scale folded into W; bit-identical to the INT8-operand kernel) when
    # the operands lie inside that kernel's exact range, which the conversions report in `o1_flag`
    o1_flag = kernels.new_range_flag(dev)
    w_bf16 = kernels.mxfp4_to_bf16_scaled(w_mxfp4, w_scale, o1_flag)
    a_bf16 = kernels.int8_to_bf16(a_int8, a_scale, o1_flag)
    o1_on_bf16 = int(o1_flag.item()) == 0
    w_sf_tiled = kernels.o2_tile_scales(w_scale)
    ws0 = kernels.FusedWorkspace("o0", M, K, dev, fuse=True)  # the one-kernel passes, timed outside the step
    ws2 = kernels.FusedWorkspace("o2", M, K, dev, fuse=True)
    a16 = torch.empty((M, K), dtype=torch.float16, device=dev)
    codes = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    sfa = torch.zeros((kernels.tiled_scale_bytes(M, K),), dtype=torch.uint8, device=dev)

    # per-variant outputs (distinct buffers so a pass's working set exceeds L2)
    y = {v: torch.empty((M, N_PER_GPU), dtype=torch.float32, device=dev) for v in VARIANTS}
    lib = kernels._lib()
    stream = torch.cuda.current_stream(dev)
    sp = stream.cuda_stream
    check = _sm100._check
    o1_gemm_name = "o1_gemm_bf16" if o1_on_bf16 else "o1_gemm_i8"
    o0_symbol = _sm100.plan_info("o0", M, N_PER_GPU, K)["kernel_symbol"]
    o2_symbol = _sm100.plan_info("o2", M, N_PER_GPU, K)["kernel_symbol"]

    def o0_conv():
        check(lib.adg_int8_to_fp16(a_int8.data_ptr(), a_scale.data_ptr(), a16.data_ptr(), M, K, sp))

    def o0_gemm():
        check(lib.adg_gemm_o0(a16.data_ptr(), w_fp16.data_ptr(), y["o0"].data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))

    def o2_conv():
        check(lib.adg_o2_quantize_activation(a_int8.data_ptr(), a_scale.data_ptr(), codes.data_ptr(), None, sfa.data_ptr(), M, K, sp))

    def o2_gemm():
        check(lib.adg_gemm_o2(codes.data_ptr(), sfa.data_ptr(), w_mxfp4.data_ptr(), w_sf_tiled.data_ptr(), y["o2"].data_ptr(),
                              M, N_PER_GPU, K, N_PER_GPU, sp))

    def o0_pass():
        check(lib.adg_o0_linear(a_int8.data_ptr(), a_scale.data_ptr(), w_fp16.data_ptr(), ws0.operand.data_ptr(),
                                ws0.counters.data_ptr(), y["o0"].data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))

    def o1_conv():
        check(lib.adg_int8_to_bf16(a_int8.data_ptr(), a_scale.data_ptr(), a_bf16.data_ptr(), o1_flag.data_ptr(), M, K, sp))

    def o1_gemm():
        if o1_on_bf16:
            check(lib.adg_gemm_o1_bf16(a_bf16.data_ptr(), a_scale.data_ptr(), w_bf16.data_ptr(), y["o1"].data_ptr(),
                                       o1_flag.data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))
        else:
            o1_int8_gemm()

    def o1_int8_gemm():
        check(lib.adg_gemm_o1(a_int8.data_ptr(), a_scale.data_ptr(), w_int8.data_ptr(), w_scale.data_ptr(),
                              y["o1"].data_ptr(), None, M, N_PER_GPU, K, N_PER_GPU, sp))

    def o2_pass():
        check(lib.adg_o2_linear(a_int8.data_ptr(), a_scale.data_ptr(), w_mxfp4.data_ptr(), w_sf_tiled.data_ptr(),
                                ws2.operand.data_ptr(), ws2.sf_tiled.data_ptr(), None, ws2.counters.data_ptr(),
                                y["o2"].data_ptr(), M, N_PER_GPU, K, N_PER_GPU, sp))

    launches = [("o0_int8_to_fp16", o0_conv), ("o0_gemm_f16", o0_gemm)] + ([("o1_int8_to_bf16", o1_conv)] if o1_on_bf16 else []) + \
               [(o1_gemm_name, o1_gemm), ("o2_quantize", o2_conv), ("o2_gemm_mxf4", o2_gemm)]

    def one_pass(events=None):
        for i, (_, fn) in enumerate(launches):
            if events is not None:
                events[i].record(stream)
            fn()
        if events is not None:
            events[len(launches)].record(stream)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if not distributed:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_passes(count: int) -> float:
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_begin.record(stream)
        for _ in range(count):
            one_pass()
        t_end.record(stream)
        barrier()
        return max_over_ranks(t_begin.elapsed_time(t_end))

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        one_pass()
    kernels.check_status(dev)
    if args.profile_pass:
        # a small target for a profiler: the six kernels of one more pass, nothing else
        one_pass()
        kernels.check_status(dev)
        print(json.dumps({"profile_pass": [name for name, _ in launches]}))
        return

    # burst: K passes from a cool start (about 10 ms)
    burst_ms = timed_passes(args.steps) / args.steps
    # passes per step so that the K timed steps last MIN_TIMED_SECONDS at the burst rate (same on every rank)
    passes_per_step = max(1, int(-(-MIN_TIMED_SECONDS * 1e3 // (burst_ms * args.steps))))
    if distributed:
        t = torch.tensor([passes_per_step], dtype=torch.int64, device=dev)
        dist.broadcast(t, src=0)
        passes_per_step = int(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    # timed region: exactly `steps` steps between two events, barrier + synchronize on both sides
    wall0 = time.perf_counter()
    total_ms = timed_passes(args.steps * passes_per_step)
    wall1 = time.perf_counter()
    # breakdown, still under load: the same passes with an event between consecutive kernels
    n_break = max(10, min(200, int(0.3e3 / burst_ms)))
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(len(launches) + 1)] for _ in range(n_break)]
    for i in range(n_break):
        one_pass(events[i])
    barrier()
    clocks = sampler.stop(window=(wall0 + 0.2, wall1)) if rank == 0 else None
    kernels.check_status(dev)
    ms_per_step = total_ms / args.steps
    ms_per_pass = ms_per_step / passes_per_step
    value = world * len(VARIANTS) * FLOP_PER_VARIANT / (ms_per_pass * 1e-3) / 1e12
    sustained_kernel_ms = {name: statistics.fmean(events[i][j].elapsed_time(events[i][j + 1]) for i in range(n_break))
                           for j, (name, _) in enumerate(launches)}
    mse = {v: float(((y[v].double() - y["o0"].double()) ** 2).mean()) for v in ("o1", "o2")}

    # ---- after a pause: per-kernel burst figures, the separate kernels the fused passes replace, conversions
    time.sleep(0.5)

    def batched(fn, reps=20):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn(0)
        torch.cuda.synchronize(dev)
        e0.record(stream)
        for i in range(reps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps

    burst_kernel_ms = {
        "o0_gemm_f16": batched(lambda i: o0_gemm()),
        o1_gemm_name: batched(lambda i: o1_gemm(), reps=10),
        "o2_gemm_mxf4": batched(lambda i: o2_gemm()),
        "o0_one_kernel": batched(lambda i: o0_pass()),
        "o2_one_kernel": batched(lambda i: o2_pass()),
    }
    if o1_on_bf16:
        y1 = y["o1"].clone()
        burst_kernel_ms["o1_gemm_i8"] = batched(lambda i: o1_int8_gemm(), reps=5)
        o1_same_bits = bool(torch.equal(y1, y["o1"]))
        del y1
    # o1x (the exact-integer O1 variant; never part of the step): GEMM-only figure and its distance from literal O1
    y1_literal = y["o1"].clone()
    o1x_weights = kernels.O1xWeights(w_mxfp4, w_scale)
    o1x_rows = o1x_weights.ineligible_rows()
    burst_kernel_ms["o1x_gemm_i8"] = batched(lambda i: kernels.gemm_o1x(a_int8, a_scale, o1x_weights, out=y["o1"]), reps=10)
    o1x_max_rel = float(((y["o1"] - y1_literal).abs() / y1_literal.abs().clamp_min(1e-3)).max())
    del y1_literal, o1x_weights
    # conversion kernels as the reference's protocol times them: batches of back-to-back launches, here rotating
    # over buffers so that the L2 does not serve them
    n_rot = 6  # 6 x (16 MiB in + 32 MiB out) > L2
    a_rot = [a_int8.clone() for _ in range(n_rot)]
    out_rot = [torch.empty((M, K), dtype=torch.float16, device=dev) for _ in range(n_rot)]
    w_rot = [w_mxfp4.clone() for _ in range(n_rot)]
    conv_ms = {
        "int8_to_fp16": batched(lambda i: check(lib.adg_int8_to_fp16(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), out_rot[i % n_rot].data_ptr(), M, K, sp)), reps=50),
        "int8_to_bf16": batched(lambda i: check(lib.adg_int8_to_bf16(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), out_rot[i % n_rot].data_ptr(), o1_flag.data_ptr(), M, K, sp)), reps=50),
        "o2_quantize": batched(lambda i: check(lib.adg_o2_quantize_activation(
            a_rot[i % n_rot].data_ptr(), a_scale.data_ptr(), out_rot[i % n_rot].data_ptr(), None, sfa.data_ptr(), M, K, sp)), reps=50),
        "mxfp4_to_fp16": batched(lambda i: check(lib.adg_mxfp4_to_fp16(
            w_rot[i % n_rot].data_ptr(), w_scale.data_ptr(), out_rot[i % n_rot].data_ptr(), N_PER_GPU, K, sp)), reps=50),
        "mxfp4_to_int8": batched(lambda i: check(lib.adg_mxfp4_to_int8(
            w_rot[i % n_rot].data_ptr(), out_rot[i % n_rot].data_ptr(), N_PER_GPU, K, sp)), reps=50),
    }
    del a_rot, out_rot, w_rot
    kernels.check_status(dev)
    torch.cuda.empty_cache()

    # ---- the N-sharded large shape, strong scaling (every rank takes part)
    sharded = sharded_block(dist, world, rank, dev)

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    conv_bytes = {"int8_to_fp16": M * K + 4 * M + 2 * M * K, "int8_to_bf16": M * K + 4 * M + 2 * M * K,
                  "o2_quantize": M * K + 4 * M + M * K // 2 + M * K // 32,
                  "mxfp4_to_fp16": N_PER_GPU * K // 2 + N_PER_GPU * K // 32 + 2 * N_PER_GPU * K,
                  "mxfp4_to_int8": N_PER_GPU * K // 2 + N_PER_GPU * K}
    # tensor peak per kernel: the measured BF16 cuBLAS figure times the MMA kind's nominal ratio to BF16
    peak_mult = {"o0_one_kernel": 1.0, "o0_gemm_f16": 1.0, "o1_gemm_bf16": 1.0, "o1_gemm_i8": 2.0, "o1x_gemm_i8": 2.0,
                 "o2_one_kernel": 4.0, "o2_gemm_mxf4": 4.0}
    nominal = {"o0_one_kernel": 2250.0, "o0_gemm_f16": 2250.0, "o1_gemm_bf16": 2250.0, "o1_gemm_i8": 4500.0, "o1x_gemm_i8": 4500.0,
               "o2_one_kernel": 9000.0, "o2_gemm_mxf4": 9000.0}
    symbols = {"o0_gemm_f16": o0_symbol, "o2_gemm_mxf4": o2_symbol, "o1_gemm_bf16": "gemm_o1_bf16_kernel", "o1_gemm_i8": "gemm_o1_kernel",
               "o0_one_kernel": _sm100.plan_info("o0", M, N_PER_GPU, K, fused=True)["kernel_symbol"],
               "o2_one_kernel": _sm100.plan_info("o2", M, N_PER_GPU, K, fused=True)["kernel_symbol"], "o1x_gemm_i8": "gemm_acc_kernel<1>",
               "o0_int8_to_fp16": "int8_to_fp16_kernel", "o1_int8_to_bf16": "int8_to_bf16_kernel", "o2_quantize": "o2_quantize_kernel"}
    step_conv_bytes = {"o0_int8_to_fp16": conv_bytes["int8_to_fp16"], "o1_int8_to_bf16": conv_bytes["int8_to_bf16"],
                       "o2_quantize": conv_bytes["o2_quantize"]}
    kernels_out = {}
    for name in sorted(set(sustained_kernel_ms) | set(burst_kernel_ms)):
        entry = {"kernel_symbol": symbols.get(name)}
        if name in peak_mult:
            for tag, ms, peak in (("sustained", sustained_kernel_ms.get(name), peaks["bf16_tflops_sustained"]),
                                  ("burst", burst_kernel_ms.get(name), peaks["bf16_tflops"])):
                if ms:
                    ach = FLOP_PER_VARIANT / (ms * 1e-3) / 1e12
                    entry[tag] = {"ms": ms, "tflops": ach, "frac_of_measured": ach / (peak * peak_mult[name]),
                                  "frac_of_nominal": ach / nominal[name]}
        else:
            ms = sustained_kernel_ms.get(name)
            nbytes = step_conv_bytes[name]
            entry["sustained"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                  "note": "inside the step, launch ramp and tail included; conversions_batched has the isolated figure"}
        kernels_out[name] = entry
    if o1_on_bf16:
        kernels_out["o1_gemm_i8"]["note"] = f"INT8-operand O1 kernel, timed outside the step; bit-identical output: {o1_same_bits}"
    for name in ("o0_one_kernel", "o2_one_kernel"):
        kernels_out[name]["note"] = "activation conversion inside the GEMM kernel (adg_o0_linear / adg_o2_linear with row counters): timed outside the step"
    kernels_out["o1x_gemm_i8"]["note"] = (f"exact-integer O1 variant, timed outside the step, never part of `value`; ineligible W rows: "
                                          f"{o1x_rows} of {N_PER_GPU}; max relative difference from literal O1: {o1x_max_rel:.2e}")
    conversions_out = {name: {"batched_ms": ms, "gbs": conv_bytes[name] / (ms * 1e-3) / 1e9,
                              "frac_of_measured_hbm": conv_bytes[name] / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              "algorithmic_bytes": conv_bytes[name]} for name, ms in conv_ms.items()}

    dominant = max((k_ for k_ in sustained_kernel_ms if k_ in peak_mult), key=sustained_kernel_ms.get)
    d_ms = sustained_kernel_ms[dominant]
    d_peak = peaks["bf16_tflops_sustained"] * peak_mult.get(dominant, 1.0)
    d_ach = FLOP_PER_VARIANT / (d_ms * 1e-3) / 1e12
    traffic = ncu_dram_traffic()
    roofline = {"kernel": dominant, "kernel_symbol": symbols.get(dominant), "bound": "tensor", "achieved": d_ach, "peak": d_peak,
                "unit": "TFLOP/s", "frac": d_ach / d_peak,
                "traffic": next((v for k_, v in traffic.items() if symbols.get(dominant, "?").split("<")[0] in k_), None),
                "traffic_source": "profiles/bench_step_kernels_full_4096.md (dram__bytes_read.sum + dram__bytes_write.sum per launch)",
                "ms": d_ms, "timed": f"average of {n_break} launches inside a sustained run (CUDA events on the launching stream)",
                "peak_source": f"{peaks['source']}: bf16 cuBLAS sustained x{peak_mult.get(dominant, 1.0):g}",
                "burst": kernels_out[dominant].get("burst")}
    if dominant in O1_ISSUE_CYCLES and clocks and clocks.get("sm_mhz"):
        partials = M * N_PER_GPU * (K // 32)
        floor_s = partials * O1_ISSUE_CYCLES[dominant] / 32 / (148 * 4 * clocks["sm_mhz"] * 1e6)
        roofline["secondary_bound"] = {
            "what": "FP32 issue slots of the epilogue: every K32 partial is scaled and accumulated separately (literal O1 "
                    f"semantics: one rounding per step and operation), {O1_ISSUE_CYCLES[dominant]:g} issue cycles per partial per warp, "
                    "at the SM clock sampled under load",
            "floor_ms": floor_s * 1e3, "frac_of_floor": floor_s * 1e3 / d_ms}

    # end to end through the host-buffer C ABI (N = 1 only): pinned A in, Y back, every variant, every pass
    e2e = None
    if not distributed:
        a_host = torch.empty((M, K), dtype=torch.int8).pin_memory()
        s_host = torch.empty((M,), dtype=torch.float32).pin_memory()
        a_host.copy_(a_int8.cpu())
        s_host.copy_(a_scale.cpu())
        y_host = {v: torch.empty((M, N_PER_GPU), dtype=torch.float32).pin_memory() for v in VARIANTS}
        w_mx_host, w_sc_host = w_mxfp4.cpu().contiguous(), w_scale.cpu().contiguous()
        sessions = {v: kernels.HostSession(v, M, w_mx_host, w_sc_host) for v in VARIANTS}
        e2e_passes = max(10, min(10 * args.steps, 100))

        def e2e_pass():
            # the three variants' passes are submitted back to back (each on its session's stream), so
            # one variant's copies overlap another's kernels; the pass ends when every Y is in host memory
            for v in VARIANTS:
                sessions[v].submit(a_host, s_host, y_host[v])
            for v in VARIANTS:
                sessions[v].wait()

        e2e_pass()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(e2e_passes):
            e2e_pass()
        e2e_sec = (time.perf_counter() - t0) / e2e_passes
        for s in sessions.values():
            s.close()
        e2e = {"value": len(VARIANTS) * FLOP_PER_VARIANT / e2e_sec / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": len(VARIANTS) * (M * K + 4 * M), "d2h_bytes_per_step": len(VARIANTS) * 4 * M * N_PER_GPU,
               "ms_per_pass": e2e_sec * 1e3, "passes": e2e_passes, "bytes_are": "per pass (one batch of activations)",
               "path": "adg_session_submit/wait (C ABI, pinned host buffers): H2D A + conversion + GEMM + D2H Y per variant, "
                       "the three variants' passes in flight together"}

    cpu = None
    if not distributed and not args.no_cpu_baseline:
        sec, kind, what = time_cpu_path(CPU_SAMPLE_ROWS, 3, 1)
        cpu = cpu_baseline_record(CPU_SAMPLE_ROWS, sec, kind, what)

    working_set = (M * K + 2 * M * K + 2 * M * K + M * K // 2) + (2 + 2 + 0.5) * N_PER_GPU * K + 3 * 4 * M * N_PER_GPU
    line = {
        "metric": "O0+O1+O2 steady-state equivalent TFLOP/s at 4096^3 (2*M*N*K per variant)",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 / bf16 (exact integers, O1) / mxf4 operands, f32 accumulate", "data": "synthetic",
        "config": {
            "workload": f"canonical M=4096 K=4096, N=4096 per GPU (W sharded by rows, global N={n_global}), steady state: "
                        "activation conversion + GEMM for O0, O1 and O2 = one pass",
            "passes_per_step": passes_per_step, "ms_per_pass": ms_per_pass, "timed_region_s": total_ms * 1e-3,
            "l2": f"no flush: each pass touches about {working_set / 2**20:.0f} MiB > 126 MiB L2",
            "seed": synthetic.CANONICAL_SEED,
            "burst": {"ms_per_pass": burst_ms, "tflops": world * len(VARIANTS) * FLOP_PER_VARIANT / (burst_ms * 1e-3) / 1e12,
                      "what": f"{args.steps} passes between two events from an idle GPU"},
            "step_kernels": [symbols.get(name, name) for name, _ in launches],
            "kernels": kernels_out,
            "conversions_batched": conversions_out,
            "mse_vs_o0": mse,
            f"sharded_{SHARDED[0]}x{SHARDED[1]}x{SHARDED[2]}": sharded,
        },
        "roofline": roofline,
        "clocks": clocks,
        "e2e": e2e,
        "cpu_baseline": cpu,
        "gpu_launches": len(launches) * (args.steps * passes_per_step),
        "timing": "value: two CUDA events around all steps (barrier + synchronize on both sides, max over ranks); "
                  "config.kernels.*.sustained: events between kernels in a run that follows the timed region without a pause; "
                  "*.burst and conversions_batched: back-to-back launches after a pause",
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
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU timing in the native arm")
    parser.add_argument("--profile-pass", action="store_true",
                        help="run the warm-up passes and ONE more pass, then exit: the target of the ncu captures under profiles/")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_native_arm(args)


if __name__ == "__main__":
    main()
