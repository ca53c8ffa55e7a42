#!/usr/bin/env python
"""Benchmark of the matmul operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1..c5] [--impl reference]

A step is one ops::matmul over one set of synthetic operands that already sit in HBM.
The default workload is configuration 2 of the baseline: bf16 A[4096,4096] @ B[4096,4096],
fp32 accumulation, bf16 result.  With N > 1 (launched by torch.distributed.run, one rank per
GPU) every rank multiplies its own 4096-row slab of a [N*4096, 4096] A by a replicated B
(weak scaling, no collective in the timed region; B is broadcast once before it).

Prints ONE JSON line (rank 0).  `value` is the whole-job TFLOP/s over the timed steps
(CUDA events on the launch stream, max over ranks).  `e2e` is the same metric through the
host-buffer entry point tvb_matmul_host: pinned host operands in, result out, copies inside
the timed region.  `roofline` relates the kernel to the measured cuBLAS bf16 peak of this
pool; `cpu_baseline` is the reference's own CPU/OpenMP ops::Mul timed on this box's cores.

`--impl reference` times the reference's CPU implementation (oracle/_ref, built from the
reference's own sources; else the C restatement in oracle/) on a bounded sample of the same
workload and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

INT8, BF16, F16, F32 = 0, 4, 5, 6
SEED_BASE = 0x5EED0000
# name: (config number, dtype, batch or None, M, K, N, dist, element size)
CONFIGS = {
    "c1": (1, F32, None, 2592, 2048, 4096, 0, 4),
    "c2": (2, BF16, None, 4096, 4096, 4096, 0, 2),
    "c3": (3, F16, 32, 1024, 4096, 1024, 0, 2),
    "c4": (4, INT8, None, 8192, 8192, 8192, 1, 1),
    "c5": (5, F32, None, 65536, 4096, 4096, 0, 4),
}
DTYPE_NAME = {INT8: "int8", BF16: "bf16", F16: "fp16", F32: "fp32"}
WORKLOAD_TEXT = {
    "c1": "fp32 A[2592,2048] @ B[2048,4096] -> fp32 (3xTF32 on tcgen05)",
    "c2": "bf16 A[4096,4096] @ B[4096,4096] -> bf16, fp32 accumulate",
    "c3": "fp16 batched A[32,1024,4096] @ B[32,4096,1024] -> fp16, fp32 accumulate",
    "c4": "int8 A[8192,8192] @ B[8192,8192] -> int8 (s32 accumulate, low byte)",
    "c5": "fp32 A[65536,4096] @ B[4096,4096] -> fp32 (3xTF32 on tcgen05)",
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the
# ncu captures summarised under profiles/ (absent = no capture of that workload yet)
NCU_TRAFFIC_BYTES = {
    "c2": 100.7e6,   # profiles/umma_gemm_pair_bf16_4096x4096x4096.md: 84.6 MB read + 16.1 MB written
    "c1": 236.1e6,   # profiles/umma_gemm_pair_counters_c1_c3_c4.md (the GEMM kernel; the split pass moves 164 MB more)
    "c3": 637.8e6,
    "c4": 390.9e6,
}
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_burst": float(d["bf16_tflops"]), "bf16_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Polls NVML (read-only) for SM clock and throttle reasons while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    if vis:
        parts = [v for v in vis.split(",") if v.strip() != ""]
        if local < len(parts) and parts[local].strip().isdigit():
            return int(parts[local])
    return local


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own ops::Mul (or the C restatement) on host cores
# ---------------------------------------------------------------------------------------------
def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use
    the host's cores (the reference itself caps its matmul at 16 threads, mul.cpp:114)."""
    n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        C.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass


def load_cpu_impl():
    """-> (kind, matmul(a, b, dtype) -> seconds, threads).  Test infrastructure under oracle/ is
    executed here, and only here, as the CPU baseline."""
    sys.path.insert(0, str(ROOT / "tests"))
    use_all_host_threads()
    import refcheck as R
    if R.have_ref():
        lib = R.ref()
        use_all_host_threads()   # again, now that the library's OpenMP runtime is loaded

        def run(a, b, dt):
            t0 = time.perf_counter()
            R.ref_matmul(a, dt, b, dt)
            return time.perf_counter() - t0
        return "reference", run, int(lib.tvref_threads()), R

    def run(a, b, dt):
        t0 = time.perf_counter()
        R.oracle_matmul(a, dt, b, dt, "cpu")
        return time.perf_counter() - t0
    return "port", run, int(R.oracle().tvo_threads()), R


def cpu_sample(R, cfg_name: str, rows: int):
    """Operands of a bounded sample: the first `rows` rows of A (of the first batches) with the
    whole B, regenerated from the configuration's seeds."""
    cfg, dt, batch, M, K, N, dist, es = CONFIGS[cfg_name]
    seed_a, seed_b = SEED_BASE + 2 * cfg, SEED_BASE + 2 * cfg + 1
    if batch is None:
        rows = min(rows, M)
        a = R.fill((rows, K), dt, seed_a, dist)
        b = R.fill((K, N), dt, seed_b, dist)
        return a, b, 2.0 * rows * K * N, f"first {rows} of {M} rows of A, whole B"
    nb = max(1, min(batch, rows // M))
    a = R.fill((nb, M, K), dt, seed_a, dist)
    b = R.fill((nb, K, N), dt, seed_b, dist)
    return a, b, 2.0 * nb * M * K * N, f"first {nb} of {batch} batches"


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0  # the CPU arm runs on rank 0 alone
    kind, run, threads, R = load_cpu_impl()
    cfg_name = args.config
    cfg, dt, batch, M, K, N, dist, es = CONFIGS[cfg_name]
    # size one step so that (steps + warmup) of them end within ~2 minutes: calibrate on the
    # smallest sample that still takes the reference's large-output path (>= 1 Mi outputs)
    budget = 120.0 / max(1, args.steps + args.warmup)
    if batch is None:
        min_rows = -(-max(64, -(-1024 * 1024 // N)) // 64) * 64
        a, b, flops, _ = cpu_sample(R, cfg_name, min_rows)
        t_probe = max(run(a, b, dt), 1e-3)
        rows = min(M, max(min_rows, int(min_rows * budget / t_probe) // 64 * 64))
    else:
        a, b, flops, _ = cpu_sample(R, cfg_name, M)          # one batch
        t_probe = max(run(a, b, dt), 1e-3)
        rows = M * min(batch, max(1, int(budget / t_probe)))
    a, b, flops, sample = cpu_sample(R, cfg_name, rows)
    for _ in range(args.warmup):
        run(a, b, dt)
    t = 0.0
    for _ in range(args.steps):
        t += run(a, b, dt)
    per = t / max(1, args.steps)
    val = flops / per / 1e12
    unit = "TOP/s" if dt == INT8 else "TFLOP/s"
    line = {
        "impl": "reference", "metric": "ops::matmul TFLOP/s", "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_NAME[dt], "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[cfg_name], "config": cfg_name,
                   "note": "reference CPU/OpenMP ops::Mul on host cores; each step is a bounded sample"},
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)

    from tensorvia_b200 import _lib, ops   # raises if the CUDA library is missing
    lib, check = _lib.lib, _lib.check
    ops.init(local)

    cfg_name = args.config
    cfg, dt, batch, M, K, N, dist_kind, es = CONFIGS[cfg_name]
    nb = batch or 1
    strong = args.scaling == "strong" and world > 1
    if strong:
        # total work fixed: this rank's rows of A (2-D) or run of batches (3-D) of the ONE problem
        if batch is None:
            begin, count = ops.shard_range(M, 128, world, rank)
            M = count
        else:
            begin, count = ops.shard_range(batch, 1, world, rank)
            nb = count
        if count == 0:
            raise SystemExit("more ranks than shards")
    seed_a, seed_b = SEED_BASE + 2 * cfg, SEED_BASE + 2 * cfg + 1
    bytes_a, bytes_b, bytes_c = nb * M * K * es, nb * K * N * es, nb * M * N * es
    flops_rank = 2.0 * nb * M * K * N

    # Rotating operand sets: successive steps touch different buffers, so that together they
    # exceed the L2 and no step finds its operands cached from the previous one.
    per_set = bytes_a + bytes_b + bytes_c
    nsets = max(2, -(-3 * L2_BYTES // per_set)) if per_set < 3 * L2_BYTES else 1
    if world > 1:
        # shards may differ by a tile row; every rank must make the same number of broadcasts below
        t = torch.tensor([nsets], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nsets = int(t[0])
    stream = torch.cuda.current_stream().cuda_stream or 1   # 1 = CUDA's handle of the legacy default stream
    sp = C.c_void_p(stream)

    def dalloc(n):
        p = C.c_void_p()
        check(lib.tvb_malloc(local, n, C.byref(p)))
        return p.value

    sets = []
    for s in range(nsets):
        pa, pb, pc = dalloc(bytes_a), dalloc(bytes_b), dalloc(bytes_c)
        # rank r owns rows [r*M, (r+1)*M) of the global A (2-D) or its own run of batches (3-D)
        first_a = (begin * (K if batch is None else M * K)) if strong else rank * nb * M * K
        check(lib.tvb_fill_splitmix(local, pa, dt, nb * M * K, seed_a + 16 * s, first_a, dist_kind, sp))
        first_b = ((begin * K * N) if strong else rank * nb * K * N) if batch else 0
        check(lib.tvb_fill_splitmix(local, pb, dt, nb * K * N, seed_b + 16 * s, first_b, dist_kind, sp))
        sets.append((pa, pb, pc))
    torch.cuda.synchronize()
    if world > 1 and batch is None:
        # "B is broadcast once": rank 0's copy goes to every rank over NCCL, outside the timed region
        for (pa, pb, pc) in sets:
            tb = torch.empty(bytes_b, dtype=torch.uint8, device="cuda")
            check(lib.tvb_memcpy_d2d(local, tb.data_ptr(), pb, bytes_b, sp))
            dist.broadcast(tb, src=0)
            check(lib.tvb_memcpy_d2d(local, pb, tb.data_ptr(), bytes_b, sp))
        torch.cuda.synchronize()

    dtc = lib.tvb_compute_type(dt, dt)

    # ---- optional gather of the row shards on rank 0 (strong scaling, 2-D problems) -----------
    gather = args.gather if (strong and batch is None) else "none"
    shared_base, gather_bufs = None, None
    if gather != "none":
        counts = [ops.shard_range(CONFIGS[cfg_name][3], 128, world, r)[1] for r in range(world)]
        full_rows = sum(counts)
    if gather == "fused":
        # rank 0 owns the whole C; every rank maps it and its GEMM epilogue stores into it over NVLink
        handle, base = _lib.IpcHandle(), C.c_void_p()
        blob = torch.zeros(C.sizeof(_lib.IpcHandle), dtype=torch.uint8, device="cuda")
        if rank == 0:
            check(lib.tvb_shared_alloc(local, full_rows * N * es, C.byref(base), C.byref(handle)))
            blob.copy_(torch.tensor(list(bytes(handle)), dtype=torch.uint8))
        dist.broadcast(blob, src=0)
        if rank != 0:
            C.memmove(C.byref(handle), bytes(blob.cpu().tolist()), C.sizeof(_lib.IpcHandle))
            check(lib.tvb_shared_open(local, C.byref(handle), C.byref(base)))
        shared_base = base.value
    elif gather == "nccl":
        tdt = {F32: torch.float32, BF16: torch.bfloat16, F16: torch.float16, INT8: torch.int8}[dt]
        c_local = torch.empty((M, N), dtype=tdt, device="cuda")
        gather_bufs = [torch.empty((n_, N), dtype=tdt, device="cuda") for n_ in counts] if rank == 0 else None

    # ---- optional: the operands as transposed views (2-D problems, one GPU) ------------------------
    # B^T ([N,K]) and / or A^T ([K,M]) are made once with tvb_transpose2d; the timed call is then
    # tvb_matmul_strided on the .t() views of those arrays, which are read in place.
    view = args.view if (world == 1 and batch is None) else "none"
    view_sets = []
    if view != "none":
        i64x3 = lambda *v: (C.c_int64 * 3)(*v)
        for (pa, pb, pc) in sets:
            va, vb = pa, pb
            sa_, sb_ = i64x3(0, K, 1), i64x3(0, N, 1)
            if view in ("at", "both"):
                va = dalloc(bytes_a)
                check(lib.tvb_transpose2d(local, pa, va, dt, M, K, sp))
                sa_ = i64x3(0, 1, M)
            if view in ("bt", "both"):
                vb = dalloc(bytes_b)
                check(lib.tvb_transpose2d(local, pb, vb, dt, K, N, sp))
                sb_ = i64x3(0, 1, K)
            view_sets.append((va, sa_, vb, sb_))
        torch.cuda.synchronize()

    def step(i):
        pa, pb, pc = sets[i % nsets]
        if view != "none":
            va, sa_, vb, sb_ = view_sets[i % nsets]
            check(lib.tvb_matmul_strided(local, va, vb, pc, dt, dt, dtc, 1, M, K, N, sa_, sb_, sp, 0))
        elif gather == "fused":
            check(lib.tvb_matmul(local, pa, pb, shared_base + begin * N * es, dt, dt, dtc, nb, M, K, N, sp))
        elif gather == "nccl":
            check(lib.tvb_matmul(local, pa, pb, c_local.data_ptr(), dt, dt, dtc, nb, M, K, N, sp))
            # gather of unequal slabs: point-to-point sends to rank 0 (what dist.gather does underneath)
            if rank == 0:
                gather_bufs[0].copy_(c_local)
                ops_ = [dist.P2POp(dist.irecv, gather_bufs[r], r) for r in range(1, world)]
            else:
                ops_ = [dist.P2POp(dist.isend, c_local, 0)]
            for w in dist.batch_isend_irecv(ops_):
                w.wait()
        else:
            check(lib.tvb_matmul(local, pa, pb, pc, dt, dt, dtc, nb, M, K, N, sp))

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    launches0 = lib.tvb_kernel_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    torch.cuda.synchronize()
    launches = lib.tvb_kernel_launches() - launches0
    clocks = sampler.stop()
    if world > 1:
        dist.barrier()
    check(lib.tvb_sync(local))  # also surfaces a timed-out device wait
    ms_total = ev0.elapsed_time(ev1)
    # minimum and median of single steps, from a second, untimed pass with an event at every step
    # boundary (the events themselves cost a few microseconds per step, so the headline figure
    # above is taken without them)
    extra = min(args.steps, 50)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(extra + 1)]
    marks[0].record()
    for i in range(extra):
        step(i)
        marks[i + 1].record()
    torch.cuda.synchronize()
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(extra))
    ms_min, ms_median = per_step[0], per_step[len(per_step) // 2]
    if world > 1:
        dist.barrier()

    # ---- end to end through the host-buffer entry point ---------------------------------------
    ha, hb, hc = C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(lib.tvb_host_alloc(bytes_a, C.byref(ha)))
    check(lib.tvb_host_alloc(bytes_b, C.byref(hb)))
    check(lib.tvb_host_alloc(bytes_c, C.byref(hc)))
    check(lib.tvb_memcpy_d2h(local, ha, sets[0][0], bytes_a, None))
    check(lib.tvb_memcpy_d2h(local, hb, sets[0][1], bytes_b, None))
    check(lib.tvb_sync(local))
    e2e_steps = max(3, min(args.steps, 50))
    for _ in range(2):
        check(lib.tvb_matmul_host(local, ha, hb, hc, dt, dt, dtc, nb, M, K, N))
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        check(lib.tvb_matmul_host(local, ha, hb, hc, dt, dt, dtc, nb, M, K, N))
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    # the result the caller got back equals the device-resident result of the same operands
    import numpy as np
    host_c = np.frombuffer((C.c_char * min(bytes_c, 1 << 20)).from_address(hc.value), dtype=np.uint8)
    dev_c = np.empty_like(host_c)
    check(lib.tvb_matmul(local, sets[0][0], sets[0][1], sets[0][2], dt, dt, dtc, nb, M, K, N, None))
    check(lib.tvb_memcpy_d2h(local, dev_c.ctypes.data, sets[0][2], dev_c.nbytes, None))
    check(lib.tvb_sync(local))
    e2e_same = bool((host_c == dev_c).all())
    if not e2e_same and dt != INT8:
        # The host call multiplies row slabs, which may run on another kernel flavour than the
        # whole problem (one CTA per tile instead of pairs, whole tiles instead of K-shared ones);
        # the flavours add the same products in different orders and may differ in the last bit.
        def as_f64(raw):
            if dt == F32:
                return raw.view(np.float32).astype(np.float64)
            if dt == F16:
                return raw.view(np.float16).astype(np.float64)
            return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        hf, df = as_f64(host_c), as_f64(dev_c)
        e2e_same = bool(np.linalg.norm(hf - df) <= (1e-5 if dt == F32 else 1e-3) * np.linalg.norm(df))
    for p in (ha, hb, hc):
        check(lib.tvb_host_free(p))

    # ---- max over ranks ---------------------------------------------------------------------------
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0]), float(t[1])
    ms_step = ms_total / args.steps
    flops_job = flops_rank * world
    if strong:
        t = torch.tensor([flops_rank], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)          # shards may differ by a tile row
        flops_job = float(t[0])
    value = flops_job / (ms_step * 1e-3) / 1e12
    e2e_value = flops_job / (e2e_ms * 1e-3) / 1e12

    if rank == 0:
        peaks = measured_peaks()
        info = ops.plan(dt, dt, nb, M, K, N, device=local)
        long_run = ms_total > 1000.0
        if dt in (BF16, F16):
            peak, peak_name = (peaks["bf16_sustained"], "bf16_tflops_sustained") if long_run else (peaks["bf16_burst"], "bf16_tflops")
        elif dt == INT8:
            peak, peak_name = 2.0 * (peaks["bf16_sustained"] if long_run else peaks["bf16_burst"]), "2 x bf16_tflops (int8 runs at twice the bf16 rate; no int8 figure was measured)"
        else:
            peak, peak_name = 0.5 * (peaks["bf16_sustained"] if long_run else peaks["bf16_burst"]) / 3.0, "bf16_tflops / 2 / 3 (tf32 runs at half the bf16 rate, three passes per product)"
        achieved = flops_rank / (ms_step * 1e-3) / 1e12
        unit = "TOP/s" if dt == INT8 else "TFLOP/s"
        line = {
            "metric": "ops::matmul TFLOP/s", "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "ms_min": ms_min, "ms_median": ms_median,
            "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": DTYPE_NAME[dt], "data": "synthetic",
            "config": {
                "workload": WORKLOAD_TEXT[cfg_name], "config": cfg_name, "per_gpu": ("1/%d of the problem per GPU" % world if strong else "one full problem per GPU") if world > 1 else "single GPU",
                "parallelism": ("rows of A sharded, B replicated" if batch is None else "batches sharded") if world > 1 else "none",
                "kernel": f"tcgen05 {info.tile_m}x{info.tile_n}x{info.tile_k}, {info.stages} stages, {info.ctas} CTAs, {info.passes} pass(es)" if info.algo == 1 else "simt",
                "l2": f"{nsets} rotating operand sets ({nsets * per_set >> 20} MiB) exceed the {L2_BYTES >> 20} MiB L2",
                "inputs": "SplitMix64 counter-based, seeds 0x5EED0000+2*cfg (A), +1 (B)",
                "view": {"none": "dense row-major operands", "bt": "B is the .t() view of a dense [N,K] array, read in place",
                         "at": "A is the .t() view of a dense [K,M] array, read in place",
                         "both": "A and B are .t() views of dense [K,M] and [N,K] arrays, read in place"}[view],
                "gather": {"none": "none: C stays sharded", "nccl": "C slabs sent to rank 0 over NCCL after each product, inside the timed region",
                           "fused": "every rank's GEMM epilogue stores its C tiles into rank 0's buffer over NVLink (peer stores), inside the timed region"}[gather],
            },
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(cfg_name), "peak_source": f"{peaks['source']}: {peak_name}",
                         "flops_per_launch": flops_rank, "frac_of_nominal_2250": (achieved / 2250.0) if dt in (BF16, F16) else None},
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": bytes_a + bytes_b, "d2h_bytes_per_step": bytes_c,
                    "ms_per_step": e2e_ms, "steps": e2e_steps, "result_equals_device_path": e2e_same,
                    "api": "tvb_matmul_host (pinned host buffers)"},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                kind, run, threads, R = load_cpu_impl()
                rows = M if batch is None else nb * M
                if cfg_name in ("c4", "c5"):
                    rows = 1024
                a, b, fl, sample = cpu_sample(R, cfg_name, rows)
                t = run(a, b, dt)
                line["cpu_baseline"] = {"value": fl / t / 1e12, "unit": unit, "cores": threads, "kind": kind,
                                        "sample": sample + f", 1 run, {t:.2f} s", "host_cpus": os.cpu_count()}
            except Exception as e:  # the baseline must never take the GPU line down
                line["cpu_baseline"] = {"value": None, "unit": unit, "cores": 0, "kind": "unavailable", "sample": str(e)[:200]}
        if world == 1 and not args.no_cpu_baseline:
            line["reference_cuda"] = reference_cuda_sample(cfg_name, unit)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def reference_cuda_sample(cfg_name: str, unit: str):
    """The reference's own CUDA kernel (mul_cuda_3d, compiled for sm_100 from its sources into
    oracle/_ref/libtv_ref_cuda.so) on the same configuration and the same GPU, in a process of its
    own, timed as the reference's tests/mul.cpp times it (wall clock around ops::Mul)."""
    lib_path = ROOT / "oracle" / "_ref" / "libtv_ref_cuda.so"
    if not lib_path.exists():
        return {"value": None, "unit": unit, "kind": "unavailable", "sample": "oracle/_ref/libtv_ref_cuda.so was not built"}
    cfg, dt, batch, M, K, N, _, _ = CONFIGS[cfg_name]
    sa = (M, K) if batch is None else (batch, M, K)
    sb = (K, N) if batch is None else (batch, K, N)
    reps = 1 if cfg_name in ("c4", "c5") else 3
    try:
        proc = subprocess.run([sys.executable, str(ROOT / "oracle" / "refcuda_run.py"), str(dt), str(dt),
                               str(SEED_BASE + 2 * cfg), str(SEED_BASE + 2 * cfg + 1), ",".join(map(str, sa)),
                               ",".join(map(str, sb)), str(reps), "-"], capture_output=True, text=True, timeout=600)
        info = json.loads(proc.stdout.strip().splitlines()[-1])
        if "error" in info:
            raise RuntimeError(info["error"])
        flops = 2.0 * (batch or 1) * M * K * N
        return {"value": flops / (info["ms_per_call"] * 1e-3) / 1e12, "unit": unit, "ms_per_call": info["ms_per_call"],
                "reps": reps, "kind": "reference CUDA backend (mul_cuda_3d, 16x16 tiles on CUDA cores) compiled for sm_100",
                "sample": "the whole configuration, ops::Mul as its tests/mul.cpp times it (result allocation and stream sync inside)"}
    except Exception as e:
        return {"value": None, "unit": unit, "kind": "unavailable", "sample": str(e)[:200]}


# ---- layout operations (secondary workloads: `--op transpose|permute|slice|concat`) --------------
# name: (what runs, elements of the source as [rows, cols] or [batch, rows, cols])
LAYOUT_TEXT = {
    "transpose": "ops::Transpose of a 2-D tensor [R, C] (tvb_transpose2d)",
    "permute": "Tensor::permute({0,2,1}).contiguous() of a batched tensor (tvb_repack)",
    "slice": "ops::Slice: the middle half of the columns of [R, C] (tvb_slice)",
    "concat": "ops::Concat along dim 1 of [R, 2C/3] and [R, C/3] (tvb_concat)",
    "typecast": "ops::Typecast bfloat16 -> float32 (tvb_typecast), the widening the reference's CPU matmul applies to half operands",
}


# (dram read + write) / algorithmic bytes of one launch, from the ncu captures of the [8192,8192]
# cases in profiles/tiled_transpose_vec_bf16_8192x8192.md; traffic grows in proportion to the tensor.
# Reads equal the source bytes in every capture; the ratio is below 1 because part of the result
# was still in the L2 when the captured (single, cold) launch ended.
NCU_LAYOUT_TRAFFIC_RATIO = {"transpose": 217.1 / 268.4, "permute": 211.4 / 268.4, "slice": 86.4 / 134.2,
                            "concat": 49.8 / 89.7, "typecast": 348.0 / 402.7}


def layout_arm(args):
    """One step = one layout operation over tensors resident in HBM; the metric is the algorithmic
    traffic (every element read once and written once) per second.  Single GPU."""
    import numpy as np
    import torch

    torch.cuda.set_device(0)
    from tensorvia_b200 import _lib, ops
    lib, check = _lib.lib, _lib.check
    ops.init(0)
    es = args.elem_bytes
    dt = {1: INT8, 2: BF16, 4: F32, 8: 3}[es]
    R_, C_ = args.rows, args.cols
    stream = torch.cuda.current_stream().cuda_stream or 1
    sp = C.c_void_p(stream)
    i64 = lambda v: (C.c_int64 * len(v))(*[int(x) for x in v])

    def dalloc(n):
        p = C.c_void_p()
        check(lib.tvb_malloc(0, n, C.byref(p)))
        return p.value

    op = args.op
    if op == "transpose":
        src_elems, dst_elems = R_ * C_, R_ * C_
        call = lambda s_, d_: lib.tvb_transpose2d(0, s_, d_, dt, R_, C_, sp)
        shape_txt = f"[{R_},{C_}] -> [{C_},{R_}]"
    elif op == "permute":
        nb, rows = 32, R_ // 32
        src_elems = dst_elems = nb * rows * C_
        shape, strides = i64([nb, C_, rows]), i64([rows * C_, 1, C_])
        call = lambda s_, d_: lib.tvb_repack(0, s_, d_, dt, 3, shape, strides, sp)
        shape_txt = f"[{nb},{rows},{C_}] viewed as [{nb},{C_},{rows}]"
    elif op == "slice":
        src_elems, dst_elems = R_ * C_, R_ * (C_ // 2)
        shape, b, e = i64([R_, C_]), i64([0, C_ // 4]), i64([R_, C_ // 4 + C_ // 2])
        call = lambda s_, d_: lib.tvb_slice(0, s_, d_, dt, 2, shape, 2, b, e, sp)
        shape_txt = f"[{R_},{C_}] -> [{R_},{C_ // 2}]"
    elif op == "typecast":
        es, dt = 2, BF16                      # source bf16, destination fp32
        src_elems = dst_elems = R_ * C_
        call = lambda s_, d_: lib.tvb_typecast(0, s_, d_, BF16, F32, R_ * C_, sp)
        shape_txt = f"[{R_},{C_}]"
    else:
        c1 = (2 * C_ // 3) // 16 * 16
        c2 = C_ - c1
        src_elems = dst_elems = R_ * C_
        shape_txt = f"[{R_},{c1}] + [{R_},{c2}] -> [{R_},{C_}]"
    des = 4 if op == "typecast" else es       # bytes per destination element
    bytes_algo = dst_elems * (es + des)       # each output element is read once and written once
    nsets = max(2, -(-3 * L2_BYTES // (src_elems * es + dst_elems * des)))
    sets = []
    for k in range(nsets):
        ps, pd = dalloc(src_elems * es), dalloc(dst_elems * des)
        check(lib.tvb_fill_splitmix(0, ps, dt, src_elems, SEED_BASE + 100 + k, 0, 1 if dt in (INT8, 3) else 0, sp))
        sets.append((ps, pd))
    if op == "concat":
        sizes, shp = i64([c1, c2]), i64([R_, c1])

        def call(s_, d_):
            ptrs = (C.c_void_p * 2)(s_, s_ + R_ * c1 * es)
            return lib.tvb_concat(0, 2, ptrs, d_, dt, 2, shp, sizes, 1, sp)
    torch.cuda.synchronize()

    def step(i):
        ps, pd = sets[i % nsets]
        check(call(ps, pd))

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    launches0 = lib.tvb_kernel_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    torch.cuda.synchronize()
    launches = lib.tvb_kernel_launches() - launches0
    clocks = sampler.stop()
    check(lib.tvb_sync(0))
    ms_step = ev0.elapsed_time(ev1) / args.steps
    gbs = bytes_algo / (ms_step * 1e-3) / 1e9

    # end to end: pinned host source in, operation, pinned host result out
    hs, hd = C.c_void_p(), C.c_void_p()
    check(lib.tvb_host_alloc(src_elems * es, C.byref(hs)))
    check(lib.tvb_host_alloc(dst_elems * des, C.byref(hd)))
    check(lib.tvb_memcpy_d2h(0, hs, sets[0][0], src_elems * es, None))
    check(lib.tvb_sync(0))
    e2e_steps = max(3, min(args.steps, 10))
    t0 = None
    for k in range(e2e_steps + 1):
        if k == 1:
            t0 = time.perf_counter()
        check(lib.tvb_memcpy_h2d(0, sets[0][0], hs, src_elems * es, sp))
        check(call(sets[0][0], sets[0][1]))
        check(lib.tvb_memcpy_d2h(0, hd, sets[0][1], dst_elems * des, sp))
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    for p_ in (hs, hd):
        check(lib.tvb_host_free(p_))

    peaks = measured_peaks()
    line = {
        "metric": "layout operation GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": f"u{8 * es}", "data": "synthetic",
        "config": {"workload": LAYOUT_TEXT[op] + " " + shape_txt, "op": op, "elem_bytes": es,
                   "l2": f"{nsets} rotating source/destination sets exceed the {L2_BYTES >> 20} MiB L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "traffic": NCU_LAYOUT_TRAFFIC_RATIO[op] * bytes_algo if es == 2 else None,
                     "traffic_note": "scaled from an ncu capture of the [8192,8192] bf16 case; reads = source bytes, part of the result still in L2 at kernel end",
                     "peak_source": f"{peaks['source']}: hbm_gbs", "bytes_per_launch": bytes_algo},
        "e2e": {"value": bytes_algo / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": src_elems * es,
                "d2h_bytes_per_step": dst_elems * des, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "api": "tvb_memcpy_h2d + the operation + tvb_memcpy_d2h (pinned host buffers)"},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        try:
            sys.path.insert(0, str(ROOT / "tests"))
            import refcheck as R
            use_all_host_threads()
            rows = min(R_, 4096)
            x = R.fill((rows, C_), dt, 1, 1 if dt in (INT8, 3) else 0)
            have = R.have_ref()
            t0 = time.perf_counter()
            if op == "transpose":
                (R.ref_transpose2d(x, dt) if have else R.oracle_transpose(x))
            elif op == "permute":
                x3 = x.reshape(32, rows // 32, C_)
                (R.ref_permute_contiguous(x3, dt, (0, 2, 1)) if have else
                 R.oracle_repack(x3, (32, C_, rows // 32), (rows // 32 * C_, 1, C_)))
            elif op == "slice":
                b_, e_ = [0, C_ // 4], [rows, C_ // 4 + C_ // 2]
                (R.ref_slice(x, dt, b_, e_) if have else R.oracle_slice(x, b_, e_))
            elif op == "typecast":
                (R.ref_typecast(x, BF16, F32) if have else R.oracle_typecast(x, BF16, F32))
            else:
                parts = [np.ascontiguousarray(x[:, :c1]), np.ascontiguousarray(x[:, c1:])]
                t0 = time.perf_counter()
                (R.ref_concat(parts, dt, 1) if have else R.oracle_concat(parts, 1))
            t = time.perf_counter() - t0
            frac = (rows / R_)
            line["cpu_baseline"] = {"value": bytes_algo * frac / t / 1e9, "unit": "GB/s", "cores": os.cpu_count() if op == "transpose" else 1,
                                    "kind": "reference" if have else "port",
                                    "sample": f"first {rows} of {R_} rows, 1 run, {t:.2f} s (includes the harness's copy of the result)"}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "unavailable", "sample": str(e)[:200]}
    emit(line)
    return 0


class OneLineStdout:
    """Routes file descriptor 1 to stderr while the benchmark runs (NCCL, the reference library
    and others print banners to stdout) and hands back the real stdout for the one JSON line."""

    def __enter__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)
        return self

    def emit(self, text: str):
        os.write(self.real, (text + "\n").encode())

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.real, 1)
        os.close(self.real)
        return False


OUT = None


def emit(line: dict):
    text = json.dumps(line)
    if OUT is not None:
        OUT.emit(text)
    else:
        print(text, flush=True)


def main():
    global OUT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="tensorvia_b200", choices=["tensorvia_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--op", default="matmul", choices=["matmul", "transpose", "permute", "slice", "concat", "typecast"],
                    help="matmul (default, the headline workload) or one of the layout operations either side of it")
    ap.add_argument("--rows", type=int, default=16384, help="layout operations: rows of the source")
    ap.add_argument("--cols", type=int, default=16384, help="layout operations: columns of the source")
    ap.add_argument("--elem-bytes", type=int, default=2, choices=[1, 2, 4, 8], help="layout operations: element size")
    ap.add_argument("--view", default="none", choices=["none", "bt", "at", "both"],
                    help="one GPU, 2-D problems: give B and / or A as transposed views (tvb_matmul_strided)")
    ap.add_argument("--gather", default="none", choices=["none", "nccl", "fused"],
                    help="with --scaling strong on a 2-D problem: also bring the whole C to rank 0 in every step")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak (default): one full problem per GPU; strong: one problem, rows or batches split over the GPUs")
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ and args.impl != "reference":
        # convenience: relaunch under torch.distributed.run, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29531", __file__] + sys.argv[1:]
        return subprocess.call(cmd)
    with OneLineStdout() as OUT:
        if args.impl == "reference":
            return reference_arm(args)
        if args.op != "matmul":
            return layout_arm(args)
        return gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
