#!/usr/bin/env python
"""Benchmark of the Roller hot path on B200: rTile search -> fp32 GEMM, README shapes M0..M13.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass over the 14 README shapes, each run by the kernel the rTile search
(plus measured feedback over its top hints, as the reference's sweep does) selected for it, in
3xTF32 mode (fp32-level accuracy). Inputs are seeded synthetic matrices, resident in HBM before
the timed region; the sweep touches ~3.2 GB per pass, so every GEMM finds its operands evicted
from the 126 MB L2. Times are CUDA-event times on the launching stream, max over ranks.

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same sweep as its row
shard of an N-times-taller GEMM (operands replicated, no data-path collective): weak scaling.
The strong-scaling shapes of the sharded configurations (8192x4096x4096 row-sharded, and
16384^3 row-sharded and on a 4x2 grid at N = 8) are timed as well and reported under "strong":
the kernels alone, with an NCCL gather of C, and with the exchange of C overlapped with the
computation.

`--impl reference` times the reference's CPU path for the same workload (numpy fp32 matmul on
the host cores + the CPU restatement of its rTile search under oracle/), rank 0 only.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import datetime
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

README_SHAPES = [
    (2048, 2048, 2048), (2048, 2048, 8192), (2048, 4096, 2048), (2048, 4096, 4096),
    (2048, 8192, 2048), (2048, 8192, 4096), (2048, 8192, 8192), (4096, 2048, 2048),
    (4096, 4096, 8192), (4096, 8192, 2048), (4096, 8192, 4096), (8192, 2048, 8192),
    (8192, 4096, 2048), (8192, 4096, 4096),
]
METRIC = "fp32 GEMM TFLOPS (README sweep M0-M13, 3xTF32, rTile-selected kernels)"
UNIT = "TFLOP/s"
WORKLOAD = "README sweep M0-M13 fp32 GEMMs, uniform[-1,1) seeded inputs, one rTile-selected kernel per shape"


def sweep_flops(shapes=README_SHAPES) -> float:
    return float(sum(2 * m * n * k for m, n, k in shapes))


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 20 ms while running. nvidia-smi
    needs a moment to start, so it is launched well before the timed region; `mark_begin` /
    `mark_end` bracket that region and only samples stamped inside it are reported."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None
        self.t_begin = None
        self.t_end = None

    def mark_begin(self):
        self.t_begin = datetime.datetime.now()

    def mark_end(self):
        self.t_end = datetime.datetime.now()

    def _inside(self, stamp: str) -> bool:
        if self.t_begin is None or self.t_end is None:
            return True
        try:
            t = datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f")
        except ValueError:
            return False
        return self.t_begin <= t <= self.t_end

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [r for r in self.rows if r and self._inside(r[0])]
        fallback = not inside and bool(self.rows)
        if fallback:            # no stamp could be matched to the region: report every sample
            inside = list(self.rows)
        for r in inside:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_outside_timed_region": len(self.rows) - len(inside),
                "power_w_median": statistics.median(power) if power else None,
                "reasons": sorted(reasons),
                **({"note": "no sample stamped inside the timed region; all samples used"}
                   if fallback else {})}


# ------------------------------------------------------------------ CPU baseline / reference arm
_blas_limit = None


def _use_all_host_threads() -> None:
    """torchrun exports OMP_NUM_THREADS=1; the CPU baseline is meant to use every host core, so
    the BLAS pool is widened again at run time."""
    global _blas_limit
    if _blas_limit is None:
        from threadpoolctl import threadpool_limits
        from oracle import gemm_oracle
        _blas_limit = threadpool_limits(limits=gemm_oracle.host_threads())


def cpu_reference_pass(shapes, budget_s: float):
    """One pass of the reference's CPU path over `shapes` (numpy fp32 matmul on all host
    threads + the search restatement), stopped once `budget_s` of matmul time is spent.
    Returns (flops done, matmul seconds, mean search ms, shapes done)."""
    from oracle import gemm_oracle, search_port
    flops, secs, done, search_ms = 0.0, 0.0, 0, []
    _use_all_host_threads()
    for i, (m, n, k) in enumerate(shapes):
        t0 = time.perf_counter()
        search_port.roller_hints(m, n, k, topk=20)
        search_ms.append((time.perf_counter() - t0) * 1e3)
        if secs >= budget_s:
            continue
        A, B = gemm_oracle.make_inputs(m, n, k, "uniform", seed=i)
        t0 = time.perf_counter()
        C = gemm_oracle.matmul_fp32(A, B)
        secs += time.perf_counter() - t0
        flops += 2.0 * m * n * k
        done += 1
        del A, B, C
    return flops, secs, statistics.mean(search_ms), done


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import gemm_oracle
    cores = gemm_oracle.host_threads()
    for _ in range(args.warmup):
        cpu_reference_pass(README_SHAPES[:1], budget_s=5.0)
    t_flops, t_secs, searches, done = 0.0, 0.0, [], 0
    for _ in range(args.steps):
        f, s, sm, d = cpu_reference_pass(README_SHAPES, budget_s=max(20.0 / args.steps, 1.0))
        t_flops += f
        t_secs += s
        searches.append(sm)
        done = d
    value = t_flops / t_secs / 1e12
    sample = (f"first {done} of the 14 README shapes per step (numpy fp32 matmul, {cores} threads), "
              f"search restatement on all 14")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample, "search_ms": statistics.mean(searches)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def measure_tf32_library_peak(torch, seconds: float = 1.0):
    """cuBLAS TF32 8192^3 through torch: (burst best-of-10, sustained over `seconds`) TFLOP/s."""
    S = 8192
    a = torch.rand(S, S, device="cuda")
    b = torch.rand(S, S, device="cuda")
    c = torch.empty(S, S, device="cuda")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for _ in range(3):
            torch.matmul(a, b, out=c)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(int(seconds * 1e3 / best), 10)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        sustained_ms = e0.elapsed_time(e1) / reps
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    fl = 2.0 * S ** 3
    return fl / best / 1e9, fl / sustained_ms / 1e9


class ShapeCase:
    """One README shape bound to its selected kernel, with resident seeded operands."""

    def __init__(self, torch, idx, shape, mode, arch, measure=True):
        from mlir_roller_b200 import roller
        from mlir_roller_b200.analyze import MatmulConfig
        self.idx, self.shape, self.mode = idx, shape, mode
        m, n, k = shape
        g = torch.Generator(device="cuda")
        g.manual_seed(idx)
        dt = roller.operand_dtype(mode)      # fp32, or bf16 / fp16 for the 16-bit modes
        self.A = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(dt)
        self.B = (torch.rand(k, n, device="cuda", generator=g) * 2 - 1).to(dt)
        self.C = torch.empty(m, n, device="cuda")
        cfg = MatmulConfig(m, n, k, 16 if dt != torch.float32 else 32)
        t0 = time.perf_counter()
        self.hint, self.fn, self.pick_ms = roller.best_hint(cfg, arch, topk=6, mode=mode,
                                                            measure=measure)
        self.select_ms = (time.perf_counter() - t0) * 1e3
        self.plan = self.fn.plan
        self.ptrs = (self.A.data_ptr(), self.B.data_ptr(), self.C.data_ptr())

    def launch(self):
        self.plan.run_ptr(*self.ptrs)

    def flops(self):
        m, n, k = self.shape
        return 2.0 * m * n * k

    def error(self, torch):
        self.launch()
        torch.cuda.synchronize()
        c64 = self.A.double() @ self.B.double()
        return float((self.C.double() - c64).abs().max() / c64.abs().max())


def measure_pcie(torch, mib: int = 512):
    """Pinned-memory copy rates of this box, GB/s: (host->device alone, device->host alone,
    each way with both directions busy). They bound the end-to-end figure."""
    n = mib * 1024 * 1024 // 4
    h_up = torch.empty(n, dtype=torch.float32).pin_memory()
    h_dn = torch.empty(n, dtype=torch.float32).pin_memory()
    d_up = torch.empty(n, device="cuda")
    d_dn = torch.empty(n, device="cuda")
    s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

    def timed(up, down, reps=3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        s_up.wait_event(e0)
        s_dn.wait_event(e0)
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s_up):
                    d_up.copy_(h_up, non_blocking=True)
            if down:
                with torch.cuda.stream(s_dn):
                    h_dn.copy_(d_dn, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s_up)
        torch.cuda.current_stream().wait_stream(s_dn)
        e1.record()
        e1.synchronize()
        return n * 4.0 * reps / e0.elapsed_time(e1) / 1e6

    timed(True, True, 1)
    return timed(True, False), timed(False, True), timed(True, True)


class LibraryCase:
    """The library GEMM (cuBLAS through torch) on a ShapeCase's operands, output in their type."""

    def __init__(self, torch, case):
        self.torch, self.A, self.B = torch, case.A, case.B
        self.C = torch.empty(case.C.shape, dtype=case.A.dtype, device="cuda")

    def launch(self):
        self.torch.matmul(self.A, self.B, out=self.C)


class SixteenBitOutCase:
    """A bf16 ShapeCase's kernel bound again with C in bf16 (what the library GEMM writes)."""

    def __init__(self, torch, case):
        from mlir_roller_b200 import _lib, roller
        m, n, k = case.shape
        self.C = torch.empty(m, n, dtype=case.A.dtype, device="cuda")
        self.plan = _lib.GemmPlan(roller.kernel_tile_for(case.hint), m, n, k, mode=case.mode,
                                  flags=_lib.FLAG_C_16BIT)
        self.ptrs = (case.A.data_ptr(), case.B.data_ptr(), self.C.data_ptr())

    def launch(self):
        self.plan.run_ptr(*self.ptrs)


def timed_sweep(torch, cases, steps, warmup, dist=None):
    """Returns (ms per step, per-shape mean ms). Barrier + synchronize on both sides."""
    for _ in range(warmup):
        for c in cases:
            c.launch()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    n = len(cases)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n + 1)] for _ in range(steps)]
    for s in range(steps):
        ev[s][0].record()
        for i, c in enumerate(cases):
            c.launch()
            ev[s][i + 1].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    total_ms = sum(ev[s][0].elapsed_time(ev[s][n]) for s in range(steps)) / steps
    per_shape = [sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(steps)) / steps
                 for i in range(n)]
    return total_ms, per_shape


def e2e_sweep(torch, cases, steps):
    """Same sweep through the host-buffer entry point: pinned host operands in, C back out,
    copies inside the timed region. Returns (ms per step, h2d bytes, d2h bytes)."""
    host = []
    for c in cases:
        hA = c.A.cpu().pin_memory()
        hB = c.B.cpu().pin_memory()
        hC = torch.empty(c.C.shape, dtype=torch.float32).pin_memory()
        host.append((hA, hB, hC))
    for c, (hA, hB, hC) in zip(cases, host):   # warm-up: allocates the plan-owned buffers
        c.plan.run_host(hA, hB, hC)
    torch.cuda.synchronize()
    # Shapes are spread over three streams so that one GEMM's upload, another's kernel and a
    # third's readback overlap (the two PCIe directions are independent); a shape always uses
    # the same stream, so its plan-owned buffers are never touched by two launches at once.
    streams = [torch.cuda.Stream() for _ in range(3)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for st in streams:
        st.wait_event(e0)
    for _ in range(steps):
        for i, (c, (hA, hB, hC)) in enumerate(zip(cases, host)):
            c.plan.run_host(hA, hB, hC, stream=streams[i % 3], wait=False)
    for st in streams:
        done = torch.cuda.Event()
        done.record(st)
        torch.cuda.current_stream().wait_event(done)
    e1.record()
    e1.synchronize()
    h2d = sum(a.numel() * 4 + b.numel() * 4 for a, b, _ in host)
    d2h = sum(c.numel() * 4 for _, _, c in host)
    checksum = float(sum(float(hc[0, 0]) for _, _, hc in host))
    return e0.elapsed_time(e1) / steps, h2d, d2h, checksum


def strong_scaling(torch, dist, rank, world, steps, warmup, mode):
    """Strong-scaling shapes of the sharded configurations. Per job: the local kernels alone
    ("compute"), followed by an NCCL gather of C to rank 0 ("with_gather"), and with the exchange
    of C running underneath the computation over symmetric memory, to rank 0
    ("overlapped_root") and to every rank ("overlapped_all"). Returns a list of records
    (identical on all ranks); times are the max over ranks."""
    from mlir_roller_b200 import mgpu
    jobs = [("M13 8192x4096x4096 row-sharded", (8192, 4096, 4096), (world, 1), 13)]
    if world == 8:
        jobs.append(("16384^3 row-sharded", (16384, 16384, 16384), (8, 1), 0))
        jobs.append(("16384^3 on a 4x2 grid", (16384, 16384, 16384), (4, 2), 0))

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = []
    for name, (M, N, K), grid, seed in jobs:
        sg = mgpu.ShardedGemm(M, N, K, rank, world, grid=grid, mode=mode, measure=True)
        b = sg.block
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        # every rank holds its rows of A and the whole (replicated) B
        A_rows = torch.rand(b.rows, K, device="cuda", generator=g) * 2 - 1
        B_full = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
        C_blk = torch.empty(b.rows, b.cols, device="cuda")
        C_full = torch.empty(M, N, device="cuda") if rank == 0 else None
        rec = {"name": name, "grid": list(grid), "tile": sg.hint.block_tile if sg.hint else None}

        def put(label, ms):
            rec[label + "_ms"] = ms
            rec[label + "_tflops"] = 2.0 * M * N * K / ms / 1e9

        put("compute", timed(lambda: sg.run(A_rows, B_full, C_blk)))
        put("with_gather", timed(lambda: (sg.run(A_rows, B_full, C_blk),
                                          sg.gather(C_blk, out=C_full))))
        del C_full
        for dest in ("root", "all"):
            try:
                og = mgpu.OverlappedGemm(M, N, K, rank, world, grid=grid, mode=mode, dest=dest)
            except Exception as e:  # noqa: BLE001 - no symmetric memory on this box: keep the rest
                rec["overlapped_error"] = f"{type(e).__name__}: {e}"[:300]
                break
            put("overlapped_" + dest, timed(lambda: (og.run(A_rows, B_full), og.finish())))
            rec["bands"] = len(og.bands)
            for p in og.plans:
                p.check_status()
            og.destroy()
            del og
            torch.cuda.empty_cache()
        # the same GEMM, unsharded, on this rank's GPU alone (the strong-scaling numerator)
        A_full = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
        C_one = torch.empty(M, N, device="cuda")
        one = mgpu.ShardedGemm(M, N, K, 0, 1, grid=(1, 1), mode=mode, measure=True)
        put("single_gpu", timed(lambda: one.run(A_full, B_full, C_one)))
        one.plan.destroy()
        del A_full, C_one, one
        torch.cuda.empty_cache()
        # lower bound of any exchange that ends with C on one rank: its ingress over NVLink
        rec["gather_link_bound_ms"] = (world - 1) / world * M * N * 4 / 770e9 * 1e3
        out.append(rec)
        del A_rows, B_full, C_blk, sg
        torch.cuda.empty_cache()
    return out


def run_gpu_arm(args) -> None:
    import torch
    from mlir_roller_b200 import _lib
    from mlir_roller_b200.analyze import (MODE_1XTF32, MODE_3XTF32, MODE_BF16, MatmulConfig,
                                          get_roller_hints)
    from mlir_roller_b200.arch import B200, CUDA

    _lib.load()  # fail loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    arch = B200.from_device(local_rank)
    sampler = ClockSampler(local_rank)     # started early: see the class
    if rank == 0:
        sampler.start()

    measure = args.select == "measure"
    cases = [ShapeCase(torch, i, s, MODE_3XTF32, arch, measure) for i, s in enumerate(README_SHAPES)]
    errs = [c.error(torch) for c in cases]
    for c in cases:
        c.plan.check_status()

    sampler.mark_begin()
    step_ms, per_shape_ms = timed_sweep(torch, cases, args.steps, args.warmup, dist)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        t = torch.tensor([step_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms = float(t.item())
    for c in cases:
        c.plan.check_status()
    value = sweep_flops() * world / step_ms / 1e9

    # 1xTF32 for the per-shape report (not part of `value`)
    cases1 = [ShapeCase(torch, i, s, MODE_1XTF32, arch, measure) for i, s in enumerate(README_SHAPES)]
    errs1 = [c.error(torch) for c in cases1]
    _, per_shape_ms1 = timed_sweep(torch, cases1, max(args.steps // 2, 1), 1, None)
    del cases1
    torch.cuda.empty_cache()

    # bf16 operands (the 16-bit kernels of the same family), with the library's bf16 GEMM timed
    # on the same operands right after; not part of `value` either
    cases16 = [ShapeCase(torch, i, s, MODE_BF16, arch, measure) for i, s in enumerate(README_SHAPES)]
    errs16 = [c.error(torch) for c in cases16]
    step_ms16, per_shape_ms16 = timed_sweep(torch, cases16, max(args.steps // 2, 1), 2, None)
    lib16 = [LibraryCase(torch, c) for c in cases16]
    step_ms16_lib, _ = timed_sweep(torch, lib16, max(args.steps // 2, 1), 2, None)
    out16 = [SixteenBitOutCase(torch, c) for c in cases16]
    step_ms16_out, _ = timed_sweep(torch, out16, max(args.steps // 2, 1), 2, None)
    for c in out16:
        c.plan.check_status()
        c.plan.destroy()
    tiles16 = [(c.hint.block_tile, c.hint.cta_group) for c in cases16]
    del cases16, lib16, out16
    torch.cuda.empty_cache()

    e2e_ms, h2d, d2h, _ = e2e_sweep(torch, cases, max(args.steps // 2, 1))
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = sweep_flops() * world / e2e_ms / 1e9

    strong = None
    if dist is not None:
        strong = strong_scaling(torch, dist, rank, world, max(args.steps // 2, 2), 2, MODE_3XTF32)

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- what the PCIe link allows for the end-to-end step: the readback runs beside the
    # upload at the duplex rate, the rest of the upload at the one-way rate
    up_gbs, down_gbs, duplex_gbs = measure_pcie(torch)
    t_down = d2h / (duplex_gbs * 1e6)
    e2e_bound_ms = t_down + max(h2d - t_down * duplex_gbs * 1e6, 0.0) / (up_gbs * 1e6)

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): algorithmic tensor flops
    # (3 TF32 products per fp32 product) per launch over the mean launch duration.
    burst_tf32, sustained_tf32 = measure_tf32_library_peak(torch)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {}
    tensor_flops = 3.0 * sweep_flops()
    achieved = tensor_flops / sum(per_shape_ms) / 1e9
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": sustained_tf32, "unit": "TFLOP/s",
        "frac": achieved / sustained_tf32,
        # DRAM bytes per launch: an ncu capture of this kernel at 4096 x 4096 x 2048 read+wrote
        # 1.13 x its algorithmic bytes 4(MK+KN+MN); scaled to the sweep's mean launch.
        "traffic": 1.13 * sum(4.0 * (m * k + k * n + m * n) for m, n, k in README_SHAPES)
        / len(README_SHAPES),
        "traffic_unit": "bytes per launch (mean over the 14 shapes), scaled from an ncu capture",
        "peak_source": ("cuBLAS TF32 8192^3 sustained, measured in this run (MEASURED_PEAKS.json "
                        "carries no TF32 entry); burst %.1f; bf16_tflops_sustained/2 = %.1f"
                        % (burst_tf32, peaks.get("bf16_tflops_sustained", 1371.6) / 2)),
        # the driver-measured file has no TF32 entry; its sustained bf16 figure halved is the
        # nearest thing to a TF32 peak it offers
        "peak_from_measured_peaks_file": peaks.get("bf16_tflops_sustained", 1371.6) / 2,
        "frac_of_measured_peaks_file": achieved / (peaks.get("bf16_tflops_sustained", 1371.6) / 2),
        "flops_per_launch": "3 * 2*M*N*K (three TF32 MMAs per fp32 product)",
        "kernel": "rb200::gemm_tf32_kernel<GemmCfg<BN,3,CG>>",
    }

    # ---- search timing: product search vs the reference's search (CPU restatement)
    from oracle import search_port
    t_new, t_ref, t_a100 = [], [], []
    for (m, n, k) in README_SHAPES:
        cfg = MatmulConfig(m, n, k, 32)
        t0 = time.perf_counter(); get_roller_hints(cfg, arch, topk=20); t_new.append(time.perf_counter() - t0)
        t0 = time.perf_counter(); get_roller_hints(cfg, CUDA(), topk=20); t_a100.append(time.perf_counter() - t0)
        t0 = time.perf_counter(); search_port.roller_hints(m, n, k, topk=20); t_ref.append(time.perf_counter() - t0)

    # ---- CPU baseline on this box's host cores (bounded sample)
    from oracle import gemm_oracle
    cpu_flops, cpu_secs, _, cpu_done = cpu_reference_pass(README_SHAPES, budget_s=15.0)
    cpu_baseline = {
        "value": cpu_flops / cpu_secs / 1e12, "unit": UNIT, "cores": gemm_oracle.host_threads(),
        "kind": "port",
        "sample": f"numpy fp32 matmul of the first {cpu_done} README shapes, one pass, all host threads",
        "search_ms_reference_port": statistics.mean(t_ref) * 1e3,
    }

    per_shape = []
    for i, (c, ms3, ms1) in enumerate(zip(cases, per_shape_ms, per_shape_ms1)):
        fl = c.flops()
        per_shape.append({
            "shape": f"M{i}", "mnk": list(c.shape), "tile": c.hint.block_tile,
            "cta_group": c.hint.cta_group,
            "ms_3x": ms3, "tflops_3x": fl / ms3 / 1e9, "frac_3x": 3 * fl / ms3 / 1e9 / sustained_tf32,
            "err_3x": errs[i],
            "ms_1x": ms1, "tflops_1x": fl / ms1 / 1e9, "frac_1x": fl / ms1 / 1e9 / sustained_tf32,
            "err_1x": errs1[i],
        })

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3 (fp32 in, fp32 accumulate/out)",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "mode": "3xTF32",
                   "l2": "inputs larger than L2: one sweep touches ~3.2 GB, L2 is 126 MB",
                   "parallelism": ("1 GPU" if world == 1 else
                                   f"{world} ranks, each the row shard of a {world}x taller GEMM, "
                                   "operands replicated, no collective")},
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "pcie_gbs": {"h2d": up_gbs, "d2h": down_gbs, "each_way_duplex": duplex_gbs},
                "pcie_bound_ms": e2e_bound_ms},
        "gpu_launches": len(cases) * args.steps,
        "search_ms": {"b200_policy": statistics.mean(t_new) * 1e3,
                      "a100_policy": statistics.mean(t_a100) * 1e3,
                      "reference_port": statistics.mean(t_ref) * 1e3},
        "max_err_3x": max(errs), "max_err_1x": max(errs1),
        "per_shape": per_shape,
        # the same sweep with bf16 operands (fp32 accumulate and C); rank 0's own GPU only
        "bf16": {
            "value": sweep_flops() / step_ms16 / 1e9, "unit": UNIT, "ms_per_step": step_ms16,
            "value_bf16_out": sweep_flops() / step_ms16_out / 1e9,   # same kernels, C in bf16
            "library_bf16_value": sweep_flops() / step_ms16_lib / 1e9,   # bf16 C
            "peak": peaks.get("bf16_tflops_sustained"),
            "frac": (sweep_flops() / step_ms16 / 1e9 / peaks["bf16_tflops_sustained"]
                     if "bf16_tflops_sustained" in peaks else None),
            "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (cuBLAS bf16 8192^3)",
            "max_err": max(errs16),
            "per_shape": [{"shape": f"M{i}", "tile": t[0], "cta_group": t[1], "ms": ms,
                           "tflops": 2.0 * m * n * k / ms / 1e9}
                          for i, ((m, n, k), t, ms) in enumerate(zip(README_SHAPES, tiles16,
                                                                     per_shape_ms16))],
        },
    }
    if strong is not None:
        line["strong"] = strong
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--select", default="measure", choices=["measure", "model"],
                    help="rTile per shape: time the top hints (default) or trust the cost model")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
