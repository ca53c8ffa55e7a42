"""Row- / batch-sharded matmul over the GPUs of one box, one process per GPU.

The reference is single-device (its CUDAContext picks one GPU,
include/backend/cuda/cuda_context.h:22-35, and Tensor::to_device ignores its device
index, src/tensor.cpp:486-509).  A matmul shards without any exchange during compute:

  2-D  C[M,N] = A[M,K] @ B[K,N]   rank r owns a contiguous slab of A's rows (a slab of the
                                  row-major buffer, no repacking) and a full copy of B
  3-D  batches are independent     rank r owns a contiguous run of batches of A, B and C

K is never split, so there is no reduction: every rank's rows are bit-identical to the
rows a single GPU would produce.  The only collectives are optional and outside the
compute: `broadcast_b` (B from one rank to all, once) and `gather_result` (all-gather of
the C slabs when one rank wants the whole result).  torch.distributed carries them (NCCL
on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from . import ops

ROW_GRANULE = 128  # rows per MMA tile: slabs are cut on tile boundaries


@dataclass(frozen=True)
class Shard:
    axis: str      # "rows" (2-D) or "batch" (3-D)
    begin: int
    count: int
    total: int


def plan(shape_a, shape_b, world: int, rank: int) -> Shard:
    """Which rows (2-D) or batches (3-D) of the problem `rank` of `world` owns."""
    batch, M, _, _ = ops.check_shapes(tuple(shape_a), tuple(shape_b))
    if len(shape_a) == 3:
        begin, count = ops.shard_range(batch, 1, world, rank)
        return Shard("batch", begin, count, batch)
    begin, count = ops.shard_range(M, ROW_GRANULE, world, rank)
    return Shard("rows", begin, count, M)


def local_shapes(shape_a, shape_b, shard: Shard):
    """Shapes of the local A, B and C buffers of a shard (None if the shard is empty)."""
    if shard.count == 0:
        return None
    if shard.axis == "batch":
        return ((shard.count, shape_a[1], shape_a[2]), (shard.count, shape_b[1], shape_b[2]),
                (shard.count, shape_a[1], shape_b[2]))
    return ((shard.count, shape_a[1]), tuple(shape_b), (shard.count, shape_b[1]))


def matmul_local(a_local, b_local, *, matmul_fn: Callable | None = None, out=None):
    """The shard's own product; `matmul_fn` defaults to the CUDA operator."""
    fn = matmul_fn or ops.matmul
    return fn(a_local, b_local, out=out) if out is not None else fn(a_local, b_local)


def broadcast_b(b, src: int = 0, group=None):
    """B from `src` to every rank (2-D problems; done once, outside any timed region)."""
    import torch.distributed as dist
    dist.broadcast(b, src=src, group=group)
    return b


def gather_result(c_local, shard: Shard, world: int, group=None):
    """All-gather of the C slabs into the full result on every rank.

    Slabs can differ in size (the last ranks may own fewer tile rows), so each rank pads its
    slab to the largest one for the collective and the padding is cut away afterwards.
    """
    import torch
    import torch.distributed as dist
    granule = ROW_GRANULE if shard.axis == "rows" else 1
    counts = [ops.shard_range(shard.total, granule, world, r)[1] for r in range(world)]
    biggest = max(counts)
    tail = tuple(c_local.shape[1:])
    padded = torch.zeros((biggest,) + tail, dtype=c_local.dtype, device=c_local.device)
    if shard.count:
        padded[: shard.count] = c_local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, counts)], dim=0)


def sharded_matmul(a_local, b_local, shard: Shard, world: int, *, gather: bool = False, group=None,
                   matmul_fn: Callable | None = None):
    """Multiplies this rank's shard; with `gather` returns the whole C on every rank."""
    c_local = matmul_local(a_local, b_local, matmul_fn=matmul_fn) if shard.count else None
    if not gather:
        return c_local
    if c_local is None:
        import torch
        n_tail = (a_local.shape[1], b_local.shape[2]) if shard.axis == "batch" else (b_local.shape[1],)
        c_local = torch.zeros((0,) + tuple(n_tail), dtype=b_local.dtype, device=b_local.device)
    return gather_result(c_local, shard, world, group=group)
