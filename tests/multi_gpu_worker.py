"""Worker of tests/test_multi_gpu.py: one rank per GPU under torch.distributed.run (NCCL).
Shards a matmul by rows (2-D) or batches (3-D), broadcasts B from rank 0 once, multiplies the
local shard with the CUDA operator, all-gathers C and compares with the unsharded product; then
repeats the product with the gather fused into the epilogue (peer stores into rank 0's buffer)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import tensorvia_b200 as tv  # noqa: E402
from tensorvia_b200 import sharded  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    ok = True
    cases = [(torch.int8, (1000, 512), (512, 768)), (torch.bfloat16, (2048, 1024), (1024, 512)),
             (torch.float32, (700, 256), (256, 300)), (torch.float16, (6, 200, 128), (6, 128, 264))]
    for dt, sa, sb in cases:
        g = torch.Generator(device="cpu").manual_seed(7)
        if dt == torch.int8:
            A = torch.randint(-10, 11, sa, generator=g, dtype=torch.int8).to(dev)
            B = torch.randint(-10, 11, sb, generator=g, dtype=torch.int8).to(dev)
        else:
            A = (torch.rand(sa, generator=g) * 2 - 1).to(dt).to(dev)
            B = (torch.rand(sb, generator=g) * 2 - 1).to(dt).to(dev)
        shard = sharded.plan(sa, sb, world, rank)
        a_loc = A[shard.begin: shard.begin + shard.count].contiguous()
        if shard.axis == "rows":
            b_loc = B.clone() if rank == 0 else torch.zeros_like(B)
            sharded.broadcast_b(b_loc, src=0)                 # B travels once, over NCCL
        else:
            b_loc = B[shard.begin: shard.begin + shard.count].contiguous()
        full = sharded.sharded_matmul(a_loc, b_loc, shard, world, gather=True)
        want = tv.matmul(A, B)
        torch.cuda.synchronize()
        if dt == torch.int8:
            good = bool((full == want).all())
        else:
            err = (torch.linalg.norm(full.double() - want.double()) / torch.linalg.norm(want.double())).item()
            good = err <= (1e-5 if dt == torch.float32 else 1e-2) and full.shape == want.shape
        ok = ok and good
        if rank == 0:
            print(f"{dt} {sa} @ {sb}: shard axis {shard.axis}, gathered {tuple(full.shape)}, match={good}", flush=True)
        # the same gather fused into the GEMM: every rank's epilogue stores into rank 0's buffer
        gathered = sharded.GatheredResult(sa, sb, dt, dt, world, rank, owner=0)
        for _ in range(2):      # the buffer is reusable
            gathered.matmul_into(a_loc, b_loc)
            whole = gathered.finish()
        if rank == 0:
            # each rank ran the kernel the unsharded problem's rows would run: bit-equal rows for
            # integers; floats may differ in the last bit where the tile plan differs
            if dt == torch.int8:
                fused_ok = bool((whole == want).all())
            else:
                err = (torch.linalg.norm(whole.double() - want.double()) / torch.linalg.norm(want.double())).item()
                fused_ok = err <= (1e-5 if dt == torch.float32 else 1e-2) and whole.shape == want.shape
            fused_ok = fused_ok and bool((whole == full).all())
            print(f"{dt} fused gather: fused_match={fused_ok}", flush=True)
            ok = ok and fused_ok
        gathered.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
