"""N-sharded execution of ``Y = A @ W.T`` over several GPUs of one node.

W's rows (the output columns) are split into contiguous, tile-aligned blocks, one per rank; each
rank holds only its slice of ``W_mxfp4`` / ``W_scale``, A and ``A_scale`` are replicated (broadcast
once), and every rank computes ``Y[:, n0:n1] = A @ W[n0:n1].T`` with the same kernels as the
single-GPU path.  K is not split, so there is no reduction and every output element is computed by
exactly the same instruction sequence as on one GPU.  A collective is needed only when a caller
wants the contiguous ``[M, N]`` result on every rank (``gather_columns``).

One process per GPU (``torchrun``); ``torch.distributed`` carries the broadcast and the optional
gather (NCCL on GPUs, gloo in the CPU tests of the partition/gather logic).
"""

from __future__ import annotations

from dataclasses import dataclass

TILE_ALIGN = 128  # shard boundaries fall on output-tile boundaries


def shard_range(n: int, world_size: int, rank: int, align: int = TILE_ALIGN) -> tuple[int, int]:
    """Rows ``[n0, n1)`` of W owned by ``rank``: blocks of ``align`` rows dealt as evenly as possible,
    earlier ranks taking the remainder; the last block may be ragged.  Empty for surplus ranks."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("invalid rank/world_size")
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world_size)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(first * align, n), min((first + count) * align, n)


def all_ranges(n: int, world_size: int, align: int = TILE_ALIGN) -> list[tuple[int, int]]:
    return [shard_range(n, world_size, r, align) for r in range(world_size)]


def broadcast_activations(a_int8, a_scale, src: int = 0, group=None):
    """Replicate A and its row scales from ``src`` (in place on the other ranks)."""
    import torch.distributed as dist

    dist.broadcast(a_int8, src=src, group=group)
    dist.broadcast(a_scale, src=src, group=group)
    return a_int8, a_scale


def gather_columns(y_local, n: int, group=None, align: int = TILE_ALIGN):
    """All-gather the ranks' column blocks ``[M, n_r]`` into the contiguous ``[M, N]`` matrix.

    Equal blocks (the usual case: N a multiple of ``align * world``) travel in ONE collective into a
    ``[world, M, N/world]`` buffer, followed by one local permute into ``[M, N]``; ragged partitions fall
    back to padded pieces."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ranges = all_ranges(n, world, align)
    m = y_local.shape[0]
    widths = {n1 - n0 for n0, n1 in ranges}
    if len(widths) == 1:
        width = widths.pop()
        stacked = torch.empty((world * m, width), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked, y_local.contiguous(), group=group)
        full = torch.empty((m, n), dtype=y_local.dtype, device=y_local.device)
        full.view(m, world, width).copy_(stacked.view(world, m, width).permute(1, 0, 2))
        return full
    widest = max(widths)
    # collectives want equal-sized pieces: ragged blocks travel padded to the widest one
    mine = y_local
    if y_local.shape[1] != widest:
        mine = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
        mine[:, : y_local.shape[1]] = y_local
    pieces = [torch.empty((m, widest), dtype=y_local.dtype, device=y_local.device) for _ in ranges]
    dist.all_gather(pieces, mine.contiguous(), group=group)
    return torch.cat([p[:, : n1 - n0] for p, (n0, n1) in zip(pieces, ranges)], dim=1)


class PeerGather:
    """Column blocks gathered by this rank's own kernel reading the other ranks' memory over NVLink.

    One process per GPU on one node.  Every rank owns ``block`` (``[M, width_r]`` FP32, the ``out=`` of its
    sharded GEMM); the allocations are exchanged once as CUDA IPC handles, and ``gather()`` runs ONE kernel
    (``adg_gather_columns_pull``) that copies every block from where it lies -- the peers' memory included --
    to its columns of a contiguous ``[M, N]``: no staging buffer and no permute pass, unlike
    ``gather_columns`` (one NCCL all-gather plus a local permute of the whole matrix).  A tiny all-reduce on
    the stream before the kernel orders it after every rank's producer, one after it keeps the blocks
    unchanged until every rank has read them."""

    def __init__(self, m: int, n: int, device, group=None, align: int = TILE_ALIGN):
        import ctypes

        import torch
        import torch.distributed as dist

        from .ops import _sm100

        self._lib = _sm100.library()
        self._sm100 = _sm100
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > _sm100.MAX_PEER_BLOCKS:
            raise RuntimeError(f"at most {_sm100.MAX_PEER_BLOCKS} ranks")
        self.m, self.n = m, n
        self.ranges = all_ranges(n, self.world, align)
        n0, n1 = self.ranges[self.rank]
        self.device = torch.device(device)
        self.block = torch.empty((m, n1 - n0), dtype=torch.float32, device=self.device)
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        handle = (ctypes.c_ubyte * _sm100.PEER_HANDLE_BYTES)()
        offset = ctypes.c_uint64(0)
        with torch.cuda.device(self.device):
            _sm100._check(self._lib.adg_peer_export(self.block.data_ptr(), handle, ctypes.byref(offset)))
        mine = (bytes(handle), int(offset.value))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._bases = {}
        self._ptrs = []
        failure = None
        for r, (peer_handle, peer_offset) in enumerate(everyone):
            if r == self.rank:
                self._ptrs.append(self.block.data_ptr())
                continue
            base = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * _sm100.PEER_HANDLE_BYTES).from_buffer_copy(peer_handle)
            with torch.cuda.device(self.device):
                if failure is None and self._lib.adg_peer_open(buf, ctypes.byref(base)) != 0:
                    failure = self._lib.adg_last_error().decode("utf-8", "replace")
            self._bases[r] = base.value
            self._ptrs.append((base.value or 0) + peer_offset)
        # all ranks agree on the outcome before anyone enters a collective that the others would not join
        ok = torch.tensor([0.0 if failure else 1.0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if float(ok.item()) == 0.0:
            for base in self._bases.values():
                if base:
                    self._lib.adg_peer_close(base)
            self._bases = {}
            raise RuntimeError(failure or "a peer could not map this rank's memory")
        # every rank starts with its right-hand neighbour, so that the links are used evenly
        order = [(self.rank + 1 + i) % self.world for i in range(self.world)]
        blocks = _sm100.PeerBlocks()
        for i, r in enumerate(order):
            blocks.src[i] = self._ptrs[r]
            blocks.col0[i] = self.ranges[r][0]
            blocks.width[i] = self.ranges[r][1] - self.ranges[r][0]
        blocks.count = self.world
        self._blocks = blocks

    def _fence(self):
        import torch.distributed as dist

        dist.all_reduce(self._token, group=self.group)

    def gather(self, out=None):
        """``[M, N]`` on every rank from the ranks' ``block`` buffers.  Stream-ordered, asynchronous."""
        import ctypes

        import torch

        full = out if out is not None else torch.empty((self.m, self.n), dtype=torch.float32, device=self.device)
        if full.shape != (self.m, self.n) or full.dtype != torch.float32 or full.stride(1) != 1:
            raise RuntimeError("out must be an [M, N] float32 matrix with unit column stride")
        self._fence()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            self._sm100._check(self._lib.adg_gather_columns_pull(ctypes.byref(self._blocks), full.data_ptr(), self.m,
                                                                 full.stride(0), stream))
        self._fence()
        return full

    def close(self):
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still be reading
        for base in self._bases.values():
            self._lib.adg_peer_close(base)
        self._bases = {}


@dataclass
class ShardedWeights:
    """One rank's slice of the weights in the forms the three variants consume."""

    n0: int
    n1: int
    w_mxfp4: object
    w_scale: object
    w_fp16: object = None    # O0
    w_int8: object = None    # O1 (INT8 operands: every input)
    o1: object = None        # O1: kernels.O1Weights (both operand forms + flag words) for kernels.o1_linear
    w_sf_tiled: object = None  # O2
    workspaces: object = None  # kernels.FusedWorkspace per variant, made on first use

    @property
    def rows(self) -> int:
        return self.n1 - self.n0


def shard_weights(w_mxfp4, w_scale, world_size: int, rank: int, variants=("o0", "o1", "o2"), device=None):
    """Slice W for ``rank`` (moving it to ``device``) and run the weight conversions once."""
    from . import kernels

    n = w_mxfp4.shape[0]
    n0, n1 = shard_range(n, world_size, rank)
    wm = w_mxfp4[n0:n1].contiguous()
    ws = w_scale[n0:n1].contiguous()
    if device is not None:
        wm, ws = wm.to(device), ws.to(device)
    shard = ShardedWeights(n0, n1, wm, ws)
    if shard.rows == 0:
        return shard
    if "o0" in variants:
        shard.w_fp16 = kernels.mxfp4_to_fp16(wm, ws)
    if "o1" in variants:
        shard.o1 = kernels.O1Weights(wm, ws)
        shard.w_int8 = shard.o1.w_int8
    if "o2" in variants:
        shard.w_sf_tiled = kernels.o2_tile_scales(ws)
    return shard


def _workspace(shard: ShardedWeights, variant: str, m: int, k: int, device, fuse: bool):
    from . import kernels

    if shard.workspaces is None:
        shard.workspaces = {}
    ws = shard.workspaces.get((variant, fuse))
    if ws is None or ws.max_m < m or ws.k != k:
        ws = shard.workspaces[(variant, fuse)] = kernels.FusedWorkspace(variant, m, k, device, fuse=fuse)
    return ws


def sharded_gemm(variant: str, a_int8, a_scale, shard: ShardedWeights, out=None, fused: bool = False):
    """This rank's column block of Y for ``variant`` (activation conversion included): the conversion of the
    replicated A, then the GEMM (``fused=True``: O0 and O2 convert A inside the GEMM kernel)."""
    from . import kernels

    if shard.rows == 0:
        return out
    m, k = a_int8.shape
    if variant == "o0":
        return kernels.o0_linear(a_int8, a_scale, shard.w_fp16, _workspace(shard, "o0", m, k, a_int8.device, fused), out=out)
    if variant == "o1":
        if getattr(shard, "o1", None) is not None:
            return kernels.o1_linear(a_int8, a_scale, shard.o1, out=out)
        return kernels.gemm_o1(a_int8, a_scale, shard.w_int8, shard.w_scale, out=out)
    if variant == "o2":
        return kernels.o2_linear(a_int8, a_scale, shard.w_mxfp4, shard.w_sf_tiled, _workspace(shard, "o2", m, k, a_int8.device, fused),
                                 out=out)
    raise ValueError(f"unknown variant: {variant}")
