"""World-size-2 test of the N-sharding plumbing on CPU ranks (gloo): partition, replicate A,
per-rank column blocks, gather.  The per-rank GEMM is stood in for by the CPU oracle, so what is
checked is that the sharded result equals the unsharded one bit for bit."""

import os
import socket

import numpy as np
import pytest

from oracle import adangel_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, out_queue):
    import torch
    import torch.distributed as dist

    from adangel_oyzl_b200 import parallel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = shape
        a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=77)
        ta, ts = torch.from_numpy(a_int8.copy()), torch.from_numpy(a_scale.copy())
        if rank != 0:  # only rank 0 holds real activations before the broadcast
            ta.zero_()
            ts.zero_()
        parallel.broadcast_activations(ta, ts, src=0)
        n0, n1 = parallel.shard_range(n, world, rank)
        block = orc.run_o1(ta.numpy(), ts.numpy(), w_mx[n0:n1], w_sc[n0:n1])["output"]
        full = parallel.gather_columns(torch.from_numpy(block), n)
        want = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
        out_queue.put((rank, bool(np.array_equal(full.numpy(), want)), (n0, n1)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(48, 512, 128), (33, 300, 64)])
def test_two_rank_sharded_result_equals_unsharded(shape):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, shape, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    ranges = dict((r, rng) for r, _, rng in results)
    assert ranges[0][1] == ranges[1][0]
