"""Strong-scaling measurement of the N-sharded GEMM (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port P \\
        -m adangel_oyzl_b200.benchmark.sharded [--m 16384 --n 28672 --k 8192] [--variants o1 o2] [--gather]

W's rows are split over the ranks (tile-aligned), A is generated on rank 0 and broadcast once (not
timed), every rank runs the same kernels on its slice, and the figure reported per variant is
``2*M*N*K`` over the slowest rank's device time (CUDA events, max over ranks).  With ``--gather`` the
all-gather of the column blocks into a contiguous Y is timed separately.  With G = 1 it runs
without a process group.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os


def main(argv=None) -> None:
    import torch

    from .. import kernels, parallel, synthetic
    from ..ops.extension import require_native

    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--m", type=int, default=16384)
    parser.add_argument("--n", type=int, default=28672)
    parser.add_argument("--k", type=int, default=8192)
    parser.add_argument("--variants", nargs="+", default=["o1", "o2"])
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--repeats", type=int, default=10)
    parser.add_argument("--gather", action="store_true")
    args = parser.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    require_native()
    m, n, k = args.m, args.n, args.k

    # activations: quantized on rank 0, replicated by one broadcast (outside every timed region)
    if rank == 0:
        g = torch.Generator().manual_seed(synthetic.CANONICAL_SEED)
        a = torch.randn(m, k, generator=g, dtype=torch.float32)
        idx = torch.randperm(k, generator=g)[: max(1, round(0.005 * k))]
        a[:, idx] *= 20.0
        a_int8, a_scale = synthetic.quantize_int8_per_row(a.to(dev))
        del a
    else:
        a_int8 = torch.empty((m, k), dtype=torch.int8, device=dev)
        a_scale = torch.empty((m,), dtype=torch.float32, device=dev)
    if dist is not None:
        parallel.broadcast_activations(a_int8, a_scale, src=0)

    # weights: every rank generates and quantizes only its own rows (seeded per rank)
    n0, n1 = parallel.shard_range(n, world, rank)
    g = torch.Generator().manual_seed(synthetic.CANONICAL_SEED + 1000 + rank)
    w = torch.randn(n1 - n0, k, generator=g, dtype=torch.float32) * 0.02
    w_mxfp4, w_scale = synthetic.quantize_mxfp4(w.to(dev))
    del w
    shard = parallel.ShardedWeights(n0, n1, w_mxfp4, w_scale)
    if "o0" in args.variants:
        shard.w_fp16 = kernels.mxfp4_to_fp16(w_mxfp4, w_scale)
    if "o1" in args.variants:
        shard.w_int8 = kernels.mxfp4_to_int8(w_mxfp4)
    if "o2" in args.variants:
        shard.w_sf_tiled = kernels.o2_tile_scales(w_scale)
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

    result = {"shape": [m, n, k], "n_gpus": world, "rows_per_rank": n1 - n0, "variants": {}}
    flop = 2.0 * m * n * k
    for variant in args.variants:
        for _ in range(args.warmup):
            parallel.sharded_gemm(variant, a_int8, a_scale, shard, out=y)
        kernels.check_status(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.repeats):
            parallel.sharded_gemm(variant, a_int8, a_scale, shard, out=y)
        e1.record()
        barrier()
        kernels.check_status(dev)
        ms = max_over_ranks(e0.elapsed_time(e1) / args.repeats)
        entry = {"steady_ms": ms, "aggregate_tflops": flop / ms / 1e9}
        if args.gather and dist is not None:
            barrier()
            e0.record()
            full = parallel.gather_columns(y, n)
            e1.record()
            barrier()
            entry["gather_ms"] = max_over_ranks(e0.elapsed_time(e1))
            entry["gathered_shape"] = list(full.shape)
            del full
        result["variants"][variant] = entry
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
