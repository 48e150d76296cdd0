"""N-sharded execution on two GPUs (NCCL): each rank computes its column block with the CUDA
kernels, the blocks are gathered, and the result must equal the single-GPU result bit for bit
(K is not split, so every element is produced by the same instruction sequence) and match the
oracle.  Skipped when fewer than two GPUs are visible."""

import os
import socket

import numpy as np
import pytest

from oracle import adangel_oracle as orc

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, queue):
    import torch
    import torch.distributed as dist

    from adangel_oyzl_b200 import kernels, parallel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        m, n, k = shape
        a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=91)
        ta = torch.from_numpy(a_int8).to(dev) if rank == 0 else torch.zeros((m, k), dtype=torch.int8, device=dev)
        ts = torch.from_numpy(a_scale).to(dev) if rank == 0 else torch.zeros((m,), dtype=torch.float32, device=dev)
        parallel.broadcast_activations(ta, ts, src=0)
        shard = parallel.shard_weights(torch.from_numpy(w_mx), torch.from_numpy(w_sc), world, rank, device=dev)
        out = {}
        peers = parallel.PeerGather(m, n, dev)
        for variant in ("o0", "o1", "o2"):
            block = parallel.sharded_gemm(variant, ta, ts, shard)
            kernels.check_status(dev)
            out[variant] = parallel.gather_columns(block, n).cpu().numpy()
            # the same blocks gathered by this rank's own kernel from the peers' memory: identical bytes
            parallel.sharded_gemm(variant, ta, ts, shard, out=peers.block)
            kernels.check_status(dev)
            pulled = peers.gather()
            torch.cuda.synchronize(dev)
            out[variant + "_pulled_equal"] = bool((pulled.cpu().numpy() == out[variant]).all())
        peers.close()
        if rank == 0:
            queue.put(out)
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_equals_single_gpu_and_oracle():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from adangel_oyzl_b200 import kernels as K

    shape = (200, 640, 512)
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, shape, queue)) for r in range(2)]
    for p in procs:
        p.start()
    sharded = queue.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(*shape, seed=91)
    da, ds, dw, dws = (torch.from_numpy(x).cuda() for x in (a_int8, a_scale, w_mx, w_sc))
    single = {
        "o0": K.gemm_o0(K.int8_to_fp16(da, ds), K.mxfp4_to_fp16(dw, dws)).cpu().numpy(),
        "o1": K.gemm_o1(da, ds, K.mxfp4_to_int8(dw), dws).cpu().numpy(),
    }
    codes, _, sfa = K.o2_quantize_activation(da, ds)
    single["o2"] = K.gemm_o2(codes, sfa, dw, K.o2_tile_scales(dws)).cpu().numpy()
    K.check_status()
    for variant in ("o0", "o1", "o2"):
        np.testing.assert_array_equal(sharded[variant], single[variant])
        assert sharded[variant + "_pulled_equal"], f"{variant}: the peer-memory gather differs from the NCCL gather"
    np.testing.assert_array_equal(sharded["o1"], orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"])
    np.testing.assert_allclose(sharded["o0"], orc.run_o0(a_int8, a_scale, w_mx, w_sc)["output"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(sharded["o2"], orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"], rtol=1e-3, atol=1e-3)
