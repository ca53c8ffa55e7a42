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

`GatheredResult` is the fused form of that gather for one rank that wants the whole result:
the owner's buffer is mapped into every rank's address space (CUDA IPC) and each rank's GEMM
writes its C tiles straight into it over NVLink from the epilogue, so there is no gather
step after the compute at all.
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


class _RawCuda:
    """Lets torch wrap a raw device pointer without copying (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class GatheredResult:
    """The whole C of a row- or batch-sharded product, living on `owner`, written by every
    rank's GEMM epilogue directly (peer stores over NVLink; no multicast, no peer loads).

    Collective: every rank of `group` constructs it with the same arguments, and calls
    `matmul_into` and `finish` the same number of times.  `tensor` is the full result on the
    owner (None elsewhere), valid after `finish`.
    """

    def __init__(self, shape_a, shape_b, dtype_a, dtype_b, world: int, rank: int, owner: int = 0, group=None):
        import ctypes as C

        import torch
        import torch.distributed as dist
        from . import _lib
        self._lib, self._dist, self._group = _lib, dist, group
        self.world, self.rank, self.owner = world, rank, owner
        to_tvb, from_tvb = ops._torch_maps()
        self.dta, self.dtb = to_tvb[dtype_a], to_tvb[dtype_b]
        self.dtc = ops.compute_type(self.dta, self.dtb)
        self.batch, self.M, self.K, self.N = ops.check_shapes(tuple(shape_a), tuple(shape_b))
        self.shard = plan(shape_a, shape_b, world, rank)
        self.shape_c = (self.batch, self.M, self.N) if len(shape_a) == 3 else (self.M, self.N)
        es = ops.dtype_size(self.dtc)
        self.nbytes = es * self.batch * self.M * self.N
        # bytes from the start of C to this rank's first row (2-D) or batch (3-D)
        self.offset = es * self.shard.begin * (self.N if self.shard.axis == "rows" else self.M * self.N)
        self.device = torch.cuda.current_device()
        ops.init(self.device)
        handle = _lib.IpcHandle()
        base = C.c_void_p()
        blob = torch.zeros(C.sizeof(_lib.IpcHandle), dtype=torch.uint8, device="cuda")
        if rank == owner:
            _lib.check(_lib.lib.tvb_shared_alloc(self.device, self.nbytes, C.byref(base), C.byref(handle)))
            blob.copy_(torch.tensor(list(bytes(handle)), dtype=torch.uint8))
        dist.broadcast(blob, src=owner, group=group)     # the handle travels once
        if rank != owner:
            C.memmove(C.byref(handle), bytes(blob.cpu().tolist()), C.sizeof(_lib.IpcHandle))
            _lib.check(_lib.lib.tvb_shared_open(self.device, C.byref(handle), C.byref(base)))
        self.base = base.value
        self.tensor = None
        if rank == owner:
            raw = torch.as_tensor(_RawCuda(self.base, self.nbytes), device="cuda")
            self.tensor = raw.view(from_tvb[self.dtc]).reshape(self.shape_c)

    def matmul_into(self, a_local, b_local):
        """This rank's shard of the product, written into the owner's buffer; asynchronous on
        torch's current stream."""
        import ctypes as C

        import torch
        if self.shard.count == 0:
            return
        if not a_local.is_contiguous() or not b_local.is_contiguous():
            raise RuntimeError("shards must be contiguous")
        stream = torch.cuda.current_stream().cuda_stream or 1
        if self.shard.axis == "rows":
            nb, m = 1, self.shard.count
        else:
            nb, m = self.shard.count, self.M
        self._lib.check(self._lib.lib.tvb_matmul(self.device, a_local.data_ptr(), b_local.data_ptr(),
                                                 self.base + self.offset, self.dta, self.dtb, self.dtc, nb, m,
                                                 self.K, self.N, C.c_void_p(stream)))

    def finish(self):
        """Waits for this rank's stores, then for every rank: after it the owner holds all of C."""
        import torch
        torch.cuda.current_stream().synchronize()
        self._dist.barrier(group=self._group)
        return self.tensor

    def close(self):
        """Collective: unmaps (peers) or frees (owner) the buffer; `tensor` must not be used after."""
        if self.base is None:
            return
        self._dist.barrier(group=self._group)      # nobody still writes
        self.tensor = None
        if self.rank == self.owner:
            self._dist.barrier(group=self._group)  # peers unmap first
            self._lib.check(self._lib.lib.tvb_shared_free(self.device, self.base))
        else:
            self._lib.check(self._lib.lib.tvb_shared_close(self.device, self.base))
            self._dist.barrier(group=self._group)
        self.base = None
