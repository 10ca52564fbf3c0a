#!/usr/bin/env python
"""Benchmark of the Roller hot path on B200: rTile search -> fp32 GEMM, README shapes M0..M13.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass over the 14 README shapes, each run by the kernel the rTile search
(plus measured feedback over its top hints, as the reference's sweep does) selected for it, in
3xTF32 mode (fp32-level accuracy). Inputs are seeded synthetic matrices, resident in HBM before
the timed region; the sweep touches ~3.2 GB per pass, so every GEMM finds its operands evicted
from the 126 MB L2. Times are CUDA-event times on the launching stream, max over ranks.

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same sweep as its row
shard of an N-times-taller GEMM (operands replicated, no data-path collective): weak scaling,
i.e. the headline `value` at N > 1 is N replicas of the sweep. The sharded configurations
(8192x4096x4096 row-sharded; 16384^3 row-sharded and on a 4x2 grid at N = 8) are timed as well
and recorded under roofline.strong: the kernels alone, with an NCCL gather of C, with the
exchange of C overlapped with the computation (copy engines, or fused into the kernel), each
with the error of the delivered C against fp64 on sampled rows.

What the driver keeps of the JSON line verbatim are the `config` and `roofline` objects, so the
per-shape table, the ragged/skinny shapes and the sharded jobs are recorded inside `roofline`.

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


_T0 = time.perf_counter()


def progress(msg: str) -> None:
    """One line on stderr (rank 0 only) with the seconds since start: where a slow run spends
    its time. stdout stays reserved for the JSON line."""
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"[bench {time.perf_counter() - _T0:7.1f}s] {msg}", file=sys.stderr, flush=True)


def sweep_flops(shapes=README_SHAPES) -> float:
    return float(sum(2 * m * n * k for m, n, k in shapes))


def workload_config(world: int) -> dict:
    """The `config` object, the same for both arms."""
    return {"workload": WORKLOAD, "mode": "3xTF32",
            "l2": "inputs larger than L2: one sweep touches ~3.2 GB, L2 is 126 MB",
            "parallelism": ("1 GPU" if world == 1 else
                            f"{world} replicas: each rank runs the sweep as the row shard of a "
                            f"{world}x taller GEMM, operands replicated, no collective; the "
                            "headline value is replica scaling, the sharded jobs are under "
                            "roofline.strong")}


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
        "data": "synthetic", "config": workload_config(args.gpus),
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
    """One shape bound to its selected kernel, with resident seeded operands."""

    def __init__(self, torch, idx, shape, mode, arch, measure=True, dist_name="uniform",
                 seed=None):
        from mlir_roller_b200 import roller
        from mlir_roller_b200.analyze import MatmulConfig
        self.torch = torch
        self.idx, self.shape, self.mode = idx, shape, mode
        m, n, k = shape
        g = torch.Generator(device="cuda")
        g.manual_seed(idx if seed is None else seed)
        dt = roller.operand_dtype(mode)      # fp32, or bf16 / fp16 for the 16-bit modes
        if dist_name == "normal":
            self.A = torch.randn(m, k, device="cuda", generator=g).to(dt)
            self.B = torch.randn(k, n, device="cuda", generator=g).to(dt)
        else:
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
        self.rotation = None

    def launch(self):
        self.plan.run_ptr(*self.ptrs)

    def flops(self):
        m, n, k = self.shape
        return 2.0 * m * n * k

    def bytes(self):
        m, n, k = self.shape
        return self.A.element_size() * (m * k + k * n) + 4.0 * m * n

    def error(self, torch):
        self.launch()
        torch.cuda.synchronize()
        c64 = self.A.double() @ self.B.double()
        return float((self.C.double() - c64).abs().max() / c64.abs().max())

    def loop_ms(self, reps, warmup=3, l2_bytes=126e6):
        """Mean ms of `reps` launches issued back to back between two events, as the
        reference times a hint (src/roller.py:564-584). Shapes whose operands would stay in
        L2 from one launch to the next rotate through copies of them (each copy bound to a
        plan of its own), so that every launch finds its operands evicted."""
        from mlir_roller_b200 import _lib, roller
        torch = self.torch
        if self.rotation is None:
            sets = max(1, int(-(-2.4 * l2_bytes // self.bytes())))
            self.rotation = [(self.plan, self.ptrs, None)]
            tile = roller.kernel_tile_for(self.hint)
            m, n, k = self.shape
            for _ in range(sets - 1):
                keep = (self.A.clone(), self.B.clone(), torch.empty_like(self.C))
                plan = _lib.GemmPlan(tile, m, n, k, mode=self.mode)
                self.rotation.append((plan, tuple(t.data_ptr() for t in keep), keep))
        rot = self.rotation
        for i in range(warmup * len(rot)):
            plan, ptrs, _ = rot[i % len(rot)]
            plan.run_ptr(*ptrs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            plan, ptrs, _ = rot[i % len(rot)]
            plan.run_ptr(*ptrs)
        e1.record()
        e1.synchronize()
        for plan, _, _ in rot:
            plan.check_status()
        return e0.elapsed_time(e1) / reps

    def release_rotation(self):
        if self.rotation:
            for plan, _, keep in self.rotation[1:]:
                plan.destroy()
        self.rotation = None


def measure_pcie(torch, mib: int = 512, only_duplex: bool = False, before=None):
    """Pinned-memory copy rates of this box, GB/s: (host->device alone, device->host alone,
    each way with both directions busy). They bound the end-to-end figure. With `only_duplex`
    just the last one is measured (returned alone), after calling `before` -- a barrier, when
    every rank of a node measures at the same moment to see what the host sustains for all
    GPUs together."""
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
    if only_duplex:
        if before is not None:
            before()
        return timed(True, True, 4)
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
    """ms per step (one pass over `cases`), launches issued back to back with an event at
    every pass boundary and nothing between the launches of a pass. Barrier + synchronize on
    both sides."""
    for _ in range(warmup):
        for c in cases:
            c.launch()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for s in range(steps):
        for c in cases:
            c.launch()
        ev[s + 1].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[steps]) / steps


def e2e_sweep(torch, cases, steps, dist=None, rank=0, world=1):
    """Same sweep from host memory: pinned host operands in, C back out, copies inside the timed
    region. Returns (ms per step, h2d bytes, d2h bytes, checksum).

    On one GPU every GEMM goes through the host-buffer entry point of the C ABI
    (roller_b200_gemm_host_async). With several ranks each rank still owns its rows of A and its
    block of C, but B is the same on all of them: a rank uploads only its 1/world share of B's
    rows and the shares are exchanged over NVLink (mgpu.HostStagedGemm), so the host links carry
    each byte of B once per node instead of once per rank."""
    from mlir_roller_b200 import mgpu, roller
    host, staged = [], []
    affinity = os.sched_getaffinity(0)
    if world > 1:
        # host buffers in the memory of the NUMA node this rank's GPU hangs off (first touch
        # while the process is restricted to that node's cores; restored below)
        mgpu.run_near_gpu(torch.cuda.current_device())
    for c in cases:
        hA = c.A.cpu().pin_memory()
        hB = c.B.cpu().pin_memory()
        hC = torch.empty(c.C.shape, dtype=torch.float32).pin_memory()
        host.append((hA, hB, hC))
        if world > 1:
            m, n, k = c.shape
            staged.append(mgpu.HostStagedGemm(m, n, k, rank, world, mode=c.mode,
                                              tile=roller.kernel_tile_for(c.hint)))
    os.sched_setaffinity(0, affinity)
    # Shapes are spread over three streams so that one GEMM's upload, another's kernel and a
    # third's readback overlap (the two PCIe directions are independent); a shape always uses
    # the same stream, so its device buffers are never touched by two launches at once.
    streams = [torch.cuda.Stream() for _ in range(3)]

    def one_pass():
        for i, (c, (hA, hB, hC)) in enumerate(zip(cases, host)):
            if world > 1:
                staged[i].run(hA, hB, hC, stream=streams[i % 3])
            else:
                c.plan.run_host(hA, hB, hC, stream=streams[i % 3], wait=False)

    one_pass()                                   # warm-up: allocates the device buffers
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for st in streams:
        st.wait_event(e0)
    for _ in range(steps):
        one_pass()
    for st in streams:
        done = torch.cuda.Event()
        done.record(st)
        torch.cuda.current_stream().wait_event(done)
    e1.record()
    e1.synchronize()
    if dist is not None:
        dist.barrier()
    if world > 1:
        moved = [g.bytes_per_call() for g in staged]
        h2d, d2h = sum(b[0] for b in moved), sum(b[1] for b in moved)
        # the staged path must deliver the same C as the kernel run on resident operands
        for c, g, (_, _, hC) in zip(cases, staged, host):
            c.launch()
            torch.cuda.synchronize()
            if not torch.equal(hC, c.C.cpu()):
                raise RuntimeError(f"end-to-end result of shape {c.shape} differs from the resident run")
            g.plan.check_status()
            g.destroy()
    else:
        h2d = sum(a.numel() * a.element_size() + b.numel() * b.element_size() for a, b, _ in host)
        d2h = sum(c.numel() * 4 for _, _, c in host)
    checksum = float(sum(float(hc[0, 0]) for _, _, hc in host))
    return e0.elapsed_time(e1) / steps, h2d, d2h, checksum


def _block_rows_operand(torch, rows, K, seed, row_block):
    """A's rows of one row block of the process grid: any rank can regenerate any block."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed * 1000 + 17 * row_block + 1)
    return torch.rand(rows, K, device="cuda", generator=g) * 2 - 1


def _sample_rows(blocks, bands_of):
    """Global rows of C to check against fp64: first and last row of every block and of every
    band a block is cut into, plus the rows either side of the first 256-row tile boundary."""
    rows = set()
    for b in blocks:
        if b.rows <= 0 or b.cols <= 0:
            continue
        rows.update((b.row0, b.row1 - 1, b.row0 + b.rows // 2))
        for r0, r1 in bands_of(b):
            rows.update((r0, r1 - 1))
        if b.rows > 256:
            rows.update((b.row0 + 255, b.row0 + 256))
    return sorted(rows)


class _Checker:
    """fp64 reference (cuBLAS DGEMM on this rank's GPU) of sampled rows of the sharded C."""

    def __init__(self, torch, blocks, grid, K, N, seed, B_full, bands_of):
        self.torch = torch
        self.rows = _sample_rows(blocks, bands_of)
        gn = grid[1]
        a_rows = []
        cache = {}
        for r in self.rows:
            b = next(x for x in blocks if x.row0 <= r < x.row1 and x.col0 == 0)
            i = b.rank // gn
            if i not in cache:
                cache[i] = _block_rows_operand(torch, b.rows, K, seed, i)
            a_rows.append(cache[i][r - b.row0])
        a = torch.stack(a_rows).double()
        del cache
        self.ref = a @ B_full.double()
        self.scale = float(self.ref.abs().max())
        self.index = torch.tensor(self.rows, device="cuda")

    def err(self, C_full):
        """max |C - ref| / max |ref| over the sampled rows of the whole M x N matrix. NaN (an
        element never written) propagates."""
        d = (C_full[self.index].double() - self.ref).abs().max()
        return float(d) / self.scale


def strong_scaling(torch, dist, rank, world, steps, warmup, budget_s=240.0, all_jobs=False,
                   fused_shapes=()):
    """The sharded configurations. Per job and mode: the local kernels alone ("kernels"), followed
    by an NCCL gather of C to rank 0 ("gather"), with the exchange of C running underneath the
    computation through the copy engines to rank 0 ("banded_root") and to every rank
    ("banded_all"), and fused into the kernel ("fused_root": the kernel's TMA unit stores the
    tiles straight into rank 0's C, progressive schedule, closed by flags; for M13 also
    "fused_root_r4" with four equal rounds and "fused_root_pipelined", the steady-state time per
    job with two C buffers on rank 0, which is a throughput and not counted as a delivery
    latency). After timing, each
    path runs once more into a NaN-filled C and the delivered matrix is compared with fp64 on
    sampled rows. Returns a list of compact records (identical on all ranks); times are the max
    over ranks, errors the max over the ranks that hold a result. Jobs that would start after
    `budget_s` seconds of this function are recorded as skipped (rank 0 decides for all), so the
    whole bench keeps to its few minutes whatever a box does."""
    from mlir_roller_b200 import mgpu
    from mlir_roller_b200.analyze import MODE_1XTF32, MODE_3XTF32
    jobs = [("M13_rows", (8192, 4096, 4096), (world, 1), 13, (MODE_3XTF32, MODE_1XTF32))]
    if world == 8:
        jobs.append(("16384_rows", (16384, 16384, 16384), (8, 1), 0, (MODE_3XTF32,)))
        jobs.append(("16384_4x2", (16384, 16384, 16384), (4, 2), 0, (MODE_3XTF32, MODE_1XTF32)))
    elif all_jobs and world % 2 == 0:
        # the 8-GPU jobs' code paths on fewer GPUs (a check of the plumbing, not a figure)
        jobs.append(("16384_rows", (16384, 16384, 16384), (world, 1), 0, (MODE_3XTF32,)))
        jobs.append((f"16384_{world // 2}x2", (16384, 16384, 16384), (world // 2, 2), 0,
                     (MODE_3XTF32, MODE_1XTF32)))

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

    def shape_of(label):
        # "fused_root_R<rounds>_<ratio>" -> (rounds, ratio); anything else: the driver's choice
        if "_R" not in label:
            return None, None
        r, q = label.split("_R")[1].split("_")
        return int(r), int(q)

    def max_over_ranks(x):
        # NaN must survive the reduction: send it as +inf
        t = torch.tensor([float("inf") if x != x else x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = []
    t_start = time.perf_counter()

    def out_of_time():
        t = torch.tensor([1.0 if time.perf_counter() - t_start > budget_s else 0.0], device="cuda")
        dist.broadcast(t, src=0)
        return bool(t.item())

    for name, (M, N, K), grid, seed, modes in jobs:
        gm, gn = grid
        if out_of_time():
            out.append({"job": name, "skipped": f"time budget of {budget_s:.0f} s used up"})
            continue
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        B_full = torch.rand(K, N, device="cuda", generator=g) * 2 - 1     # replicated
        for mode in modes:
            if out_of_time():
                out.append({"job": name, "mode": f"{mode}xTF32",
                            "skipped": f"time budget of {budget_s:.0f} s used up"})
                continue
            progress(f"strong: {name} mode {mode} on {gm}x{gn}")
            sg = mgpu.ShardedGemm(M, N, K, rank, world, grid=grid, mode=mode, measure=True)
            b = sg.block
            A_rows = _block_rows_operand(torch, b.rows, K, seed, rank // gn)
            C_blk = torch.empty(b.rows, b.cols, device="cuda")
            C_full = torch.empty(M, N, device="cuda") if rank == 0 else None
            rec = {"job": name, "mode": f"{mode}xTF32", "grid": f"{gm}x{gn}",
                   "tile": "x".join(str(v) for v in (sg.hint.block_tile if sg.hint else []))}
            flops = 2.0 * M * N * K

            rec["kernels_ms"] = timed(lambda: sg.run(A_rows, B_full, C_blk))
            rec["gather_ms"] = timed(lambda: (sg.run(A_rows, B_full, C_blk),
                                              sg.gather(C_blk, out=C_full)))
            # (the exchanges over symmetric memory: a box that cannot provide it keeps the figures
            # above and records the reason; the failure must be the same on every rank, which an
            # allocation or rendezvous failure is)
            try:
                ob = mgpu.OverlappedGemm(M, N, K, rank, world, grid=grid, mode=mode, dest="root")
                n_bands = len(ob.bands)
            except Exception as e:  # noqa: BLE001
                ob, n_bands = None, 1
                rec["overlapped_error"] = f"{type(e).__name__}: {e}"[:200]
            checker = _Checker(torch, sg.blocks, grid, K, N, seed, B_full,
                               lambda blk: mgpu.split_bands(blk.row0, blk.row1, n_bands))
            # the gathered C of the run above (rank 0 holds it)
            if rank == 0:
                C_full.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            sg.run(A_rows, B_full, C_blk)
            sg.gather(C_blk, out=C_full)
            torch.cuda.synchronize()
            rec["gather_err"] = max_over_ranks(checker.err(C_full) if rank == 0 else 0.0)
            del C_full
            sg.plan.check_status()

            paths = [("banded_root", ob, False), ("banded_all", None, True), ("fused_root", None, False)]
            if ob is None:
                paths = []
            elif name.startswith("M13"):
                # for comparison: four equal rounds instead of the geometric sequence the
                # driver derives from t_link / t_compute
                paths.append(("fused_root_r4", None, False))
                # two C buffers on rank 0: a sender starts step s + 1 while rank 0 may still read
                # step s, so the steady-state time per job is what is timed, not a latency
                paths.append(("fused_root_pipelined", None, False))
                # (--fused-shapes: other round counts and ratios of the progressive schedule)
                paths.extend((f"fused_root_R{r}_{q}", None, False) for r, q in fused_shapes)
            for label, og, everywhere in paths:
                try:
                    if og is None:
                        og = mgpu.OverlappedGemm(M, N, K, rank, world, grid=grid, mode=mode,
                                                 dest="all" if everywhere else "root",
                                                 fused=label.startswith("fused_root"),
                                                 depth=2 if label.endswith("_pipelined") else 1,
                                                 rounds=4 if label.endswith("_r4") else shape_of(label)[0],
                                                 round_ratio=100 if label.endswith("_r4") else shape_of(label)[1])
                except Exception as e:  # noqa: BLE001 - keep the other paths' numbers
                    rec[label + "_error"] = f"{type(e).__name__}: {e}"[:200]
                    continue
                progress(f"strong: {name} mode {mode}: {label}")
                rec[label + "_ms"] = timed(lambda: (og.run(A_rows, B_full), og.finish()))
                for c_buf in og.C_bufs:
                    c_buf.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                og.run(A_rows, B_full)
                og.finish()
                torch.cuda.synchronize()
                dist.barrier()
                og.check_status()
                holds = everywhere or rank == 0
                rec[label + "_err"] = max_over_ranks(checker.err(og.C) if holds else 0.0)
                if label == "banded_root":
                    rec["bands"] = len(og.bands)
                if label.startswith("fused_root") and og.plans:
                    info = og.plans[0].schedule_info()
                    # (the sending ranks' schedule; rank 0 keeps C at home and runs whole tiles)
                    rec[label.replace("fused_root", "fused_rounds")] = int(
                        max_over_ranks(float(info["rounds"]) if rank != 0 else 0.0))
                    rec[label.replace("fused_root", "fused_ratio")] = int(
                        max_over_ranks(float(og.round_ratio or 0) if rank != 0 else 0.0))
                og.destroy()
                del og
                torch.cuda.empty_cache()
            del checker
            # the same GEMM, unsharded, on this rank's GPU alone (the strong-scaling numerator)
            progress(f"strong: {name} mode {mode}: single GPU")
            A_full = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
            C_one = torch.empty(M, N, device="cuda")
            one = mgpu.ShardedGemm(M, N, K, 0, 1, grid=(1, 1), mode=mode, measure=True)
            rec["single_ms"] = timed(lambda: one.run(A_full, B_full, C_one))
            one.plan.destroy()
            del A_full, C_one, one
            torch.cuda.empty_cache()
            # lower bound of any exchange that ends with C on one rank: its NVLink ingress at the
            # measured 770 GB/s per direction
            link_ms = (world - 1) / world * M * N * 4 / 770e9 * 1e3
            rec["link_bound_ms"] = link_ms
            # (the latency of one job: the pipelined form is a throughput and is kept apart)
            best_root = min(v for k, v in rec.items() if k.endswith("_ms") and
                            k.startswith(("banded_root", "fused_root", "gather")) and
                            "pipelined" not in k)
            if "fused_root_pipelined_ms" in rec:
                rec["eff_pipelined_root"] = rec["single_ms"] / (world * rec["fused_root_pipelined_ms"])
            rec["delivered_root_ms"] = best_root
            rec["ingress_gbs"] = (world - 1) / world * M * N * 4 / best_root / 1e6
            rec["eff_kernels"] = rec["single_ms"] / (world * rec["kernels_ms"])
            rec["eff_delivered_root"] = rec["single_ms"] / (world * best_root)
            rec["eff_ceiling"] = rec["single_ms"] / (world * max(link_ms, rec["kernels_ms"]))
            rec["tflops_delivered_root"] = flops / best_root / 1e9
            out.append({k: (round(v, 5) if isinstance(v, float) and v == v and abs(v) < 1e30
                            and k.endswith(("_ms", "_gbs")) else v) for k, v in rec.items()})
            sg.plan.destroy()
            del A_rows, C_blk, sg
            torch.cuda.empty_cache()
        del B_full
        torch.cuda.empty_cache()
    return out


CONFIG4_SHAPES = [("ragged", (4097, 2049, 8193)), ("skinny", (16, 8192, 8192))]
HBM_GBS_FALLBACK = 6650.0


def config4_records(torch, arch, peak_tf32, hbm_gbs, reps):
    """The ragged and the skinny GEMM (normal(0,1) inputs, seed 0), both modes: time per launch in
    a back-to-back loop, fraction of t_roof = max(flops / P_tf32, bytes / BW_hbm), error against
    fp64. For the ragged shape, whose rows are not multiples of 16 bytes, the same kernel is
    also timed on operands that were padded beforehand: the difference is what the two staging
    copies inside every launch cost."""
    from mlir_roller_b200 import _lib, roller
    from mlir_roller_b200.analyze import MODE_1XTF32, MODE_3XTF32
    out = []
    for name, shape in CONFIG4_SHAPES:
        m, n, k = shape
        for mode in (MODE_3XTF32, MODE_1XTF32):
            case = ShapeCase(torch, 0, shape, mode, arch, True, dist_name="normal", seed=0)
            err = case.error(torch)
            ms = case.loop_ms(reps)
            flops = (3 if mode == MODE_3XTF32 else 1) * 2.0 * m * n * k
            t_roof_ms = max(flops / (peak_tf32 * 1e9), case.bytes() / (hbm_gbs * 1e6))
            rec = {"shape": name, "mnk": list(shape), "mode": f"{mode}xTF32",
                   "tile": "x".join(str(v) for v in case.hint.block_tile) + f"/cg{case.hint.cta_group}"
                           + ("/skinny" if getattr(case.hint, "layout", 0) == 2 else ""),
                   "us": ms * 1e3, "frac_of_t_roof": t_roof_ms / ms,
                   "bound": "tensor" if flops / (peak_tf32 * 1e9) >= case.bytes() / (hbm_gbs * 1e6)
                   else "hbm",
                   "tflops": 2.0 * m * n * k / ms / 1e9, "gbs": case.bytes() / ms / 1e6, "err": err}
            if k % 4 or n % 4:
                # the same product with the operands padded once, outside the timed loop
                kp, np_ = -(-k // 4) * 4, -(-n // 4) * 4
                Ap = torch.zeros(m, kp, device="cuda"); Ap[:, :k] = case.A
                Bp = torch.zeros(k, np_, device="cuda"); Bp[:, :n] = case.B
                Cp = torch.empty(m, np_, device="cuda")
                plan = _lib.GemmPlan(roller.kernel_tile_for(case.hint), m, n, k, lda=kp, ldb=np_,
                                     ldc=np_, mode=mode)
                ms_aligned = plan.time(Ap, Bp, Cp, warmup=3, iters=reps)
                plan.check_status()
                plan.destroy()
                rec["us_operands_prepadded"] = ms_aligned * 1e3
                rec["staging_copies_share"] = max(0.0, 1.0 - ms_aligned / ms)
                del Ap, Bp, Cp
            case.release_rotation()
            case.plan.destroy()
            del case
            torch.cuda.empty_cache()
            out.append(rec)
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
    parts = set(args.parts.split(","))
    progress(f"start, world {world}")
    cases = [ShapeCase(torch, i, s, MODE_3XTF32, arch, measure) for i, s in enumerate(README_SHAPES)]
    errs = [c.error(torch) for c in cases]
    for c in cases:
        c.plan.check_status()

    progress("kernels selected, timing the sweep")
    sampler.mark_begin()
    step_ms = timed_sweep(torch, cases, args.steps, args.warmup, dist)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        t = torch.tensor([step_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms = float(t.item())
    for c in cases:
        c.plan.check_status()
    value = sweep_flops() * world / step_ms / 1e9

    # Per-shape table, both modes: each shape in a back-to-back loop of its own (rank 0's GPU is
    # enough: every rank runs the same kernels on the same shapes).
    loop_reps = max(args.steps, 10)
    per_shape_ms = per_shape_ms1 = errs1 = tiles1 = None
    step_ms16 = None
    progress("sweep timed; per-shape loops, 1xTF32 and bf16 on rank 0")
    if rank == 0:
        per_shape_ms = [c.loop_ms(loop_reps) for c in cases]
        for c in cases:
            c.release_rotation()
        torch.cuda.empty_cache()
        cases1 = [ShapeCase(torch, i, s, MODE_1XTF32, arch, measure)
                  for i, s in enumerate(README_SHAPES)]
        errs1 = [c.error(torch) for c in cases1]
        per_shape_ms1 = [c.loop_ms(loop_reps) for c in cases1]
        tiles1 = [(c.hint.block_tile, c.hint.cta_group) for c in cases1]
        for c in cases1:
            c.release_rotation()
            c.plan.destroy()
        del cases1
        torch.cuda.empty_cache()

        # bf16 operands (the 16-bit kernels of the same family), with the library's bf16 GEMM
        # timed on the same operands right after; not part of `value` either
        cases16 = [ShapeCase(torch, i, s, MODE_BF16, arch, measure)
                   for i, s in enumerate(README_SHAPES)]
        errs16 = [c.error(torch) for c in cases16]
        half = max(args.steps // 2, 1)
        step_ms16 = timed_sweep(torch, cases16, half, 2, None)
        lib16 = [LibraryCase(torch, c) for c in cases16]
        step_ms16_lib = timed_sweep(torch, lib16, half, 2, None)
        out16 = [SixteenBitOutCase(torch, c) for c in cases16]
        step_ms16_out = timed_sweep(torch, out16, half, 2, None)
        for c in out16:
            c.plan.check_status()
            c.plan.destroy()
        tiles16 = [(c.hint.block_tile, c.hint.cta_group) for c in cases16]
        for c in cases16:
            c.plan.destroy()
        del cases16, lib16, out16
        torch.cuda.empty_cache()

    progress("end-to-end sweep from host memory")
    e2e_ms, h2d, d2h, _ = e2e_sweep(torch, cases, max(args.steps // 2, 1), dist, rank, world)
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = sweep_flops() * world / e2e_ms / 1e9
    tiles3 = [(c.hint.block_tile, c.hint.cta_group) for c in cases]
    for c in cases:
        c.plan.destroy()
    del cases
    torch.cuda.empty_cache()

    strong = None
    if dist is not None and "strong" in parts:
        progress("sharded jobs")
        strong = strong_scaling(torch, dist, rank, world, max(args.steps // 2, 3), 2,
                                budget_s=args.strong_budget_s, all_jobs="alljobs" in parts,
                                fused_shapes=[tuple(int(v) for v in s.split(":"))
                                              for s in args.fused_shapes.split(",") if s])
    # what the host sustains when every GPU of the node copies both ways at once (the slowest
    # rank's rate): the end-to-end step of N ranks cannot beat it
    duplex_all_gbs = None
    if dist is not None:
        mine = measure_pcie(torch, mib=256, only_duplex=True, before=dist.barrier)
        t = torch.tensor([mine], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        duplex_all_gbs = float(t.item())
    progress("measurements done on all ranks")

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
    pcie = {"h2d": up_gbs, "d2h": down_gbs, "each_way_duplex": duplex_gbs}
    if duplex_all_gbs is not None:
        # with all ranks copying: the same estimate with the duplex rate the host then sustains
        pcie["each_way_duplex_all_ranks_at_once"] = duplex_all_gbs
        t_down = d2h / (duplex_all_gbs * 1e6)
        e2e_bound_ms = max(e2e_bound_ms,
                           t_down + max(h2d - t_down * duplex_all_gbs * 1e6, 0.0) / (up_gbs * 1e6))

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): algorithmic tensor flops (3 TF32
    # products per fp32 product) of one step over the step's duration. The denominator is a
    # library TF32 GEMM measured in this run (the driver-written peaks file has no TF32 entry)
    # in the regime the timed region ran in: the best single launch ("burst") for a region
    # shorter than a second -- the GPU has not reached its power-capped steady state by then --
    # and the rate sustained over a second otherwise. The bf16 figures of the peaks file,
    # halved, are printed beside it.
    burst_tf32, sustained_tf32 = measure_tf32_library_peak(torch)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {}
    hbm_gbs = float(peaks.get("hbm_gbs", HBM_GBS_FALLBACK))
    region_s = step_ms * args.steps / 1e3
    burst_regime = region_s < 1.0
    peak = burst_tf32 if burst_regime else sustained_tf32
    if "bf16_tflops" in peaks and burst_regime:
        peak = max(peak, peaks["bf16_tflops"] / 2)       # never a softer denominator than the file's
    tensor_flops = 3.0 * sweep_flops()
    achieved = tensor_flops / step_ms / 1e9
    shape_peak = max(burst_tf32, peaks.get("bf16_tflops", 0.0) / 2)   # loops of a few ms: burst

    per_shape = []
    for i, (shape, ms3, ms1) in enumerate(zip(README_SHAPES, per_shape_ms, per_shape_ms1)):
        fl = 2.0 * shape[0] * shape[1] * shape[2]
        per_shape.append({
            "s": f"M{i}", "tile3": "x".join(map(str, tiles3[i][0])) + f"/cg{tiles3[i][1]}",
            "us3": round(ms3 * 1e3, 2), "tf3": round(fl / ms3 / 1e9, 1),
            "frac3": round(3 * fl / ms3 / 1e9 / shape_peak, 4), "err3": float(f"{errs[i]:.3g}"),
            "tile1": "x".join(map(str, tiles1[i][0])) + f"/cg{tiles1[i][1]}",
            "us1": round(ms1 * 1e3, 2), "tf1": round(fl / ms1 / 1e9, 1),
            "frac1": round(fl / ms1 / 1e9 / shape_peak, 4), "err1": float(f"{errs1[i]:.3g}"),
        })
    config4 = config4_records(torch, arch, shape_peak, hbm_gbs, loop_reps)

    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak,
        # DRAM bytes per launch: an ncu capture of this kernel at 4096 x 4096 x 2048 read+wrote
        # 1.18 x its algorithmic bytes 4(MK+KN+MN); scaled to the sweep's mean launch.
        "traffic": 1.18 * sum(4.0 * (m * k + k * n + m * n) for m, n, k in README_SHAPES)
        / len(README_SHAPES),
        "traffic_unit": "bytes per launch (mean over the 14 shapes), scaled from an ncu capture",
        "peak_regime": "burst" if burst_regime else "sustained",
        "peak_source": ("library TF32 GEMM (cuBLAS through torch, 8192^3) measured in this run: "
                        "burst %.1f, sustained over 1 s %.1f TFLOP/s; the timed region lasted "
                        "%.2f s, so the %s figure is the denominator. MEASURED_PEAKS.json has no "
                        "TF32 entry; its bf16 figures halved: burst %.1f, sustained %.1f"
                        % (burst_tf32, sustained_tf32, region_s,
                           "burst" if burst_regime else "sustained",
                           peaks.get("bf16_tflops", float("nan")) / 2,
                           peaks.get("bf16_tflops_sustained", float("nan")) / 2)),
        "peak_tf32_burst": burst_tf32, "peak_tf32_sustained": sustained_tf32,
        "frac_of_sustained": achieved / sustained_tf32,
        "flops_per_launch": "3 * 2*M*N*K (three TF32 MMAs per fp32 product)",
        "kernel": "rb200::gemm_tf32_kernel<GemmCfg<BN,3,CG>>",
        "timed_region_s": region_s,
        # per README shape, back-to-back loops of one shape each; frac = tensor flops / time /
        # the burst peak (3x counted at 3 x 2MNK); err = max|C - C64| / max|C64|
        "per_shape": per_shape,
        "per_shape_min_frac3": min(r["frac3"] for r in per_shape),
        "per_shape_min_frac1": min(r["frac1"] for r in per_shape),
        "per_shape_peak": shape_peak,
        "max_err_3x": max(errs), "max_err_1x": max(errs1),
        # the ragged and the skinny GEMM of the tail / memory-bound configuration
        "config4": config4,
        "hbm_gbs_peak": hbm_gbs,
    }
    if strong is not None:
        roofline["strong"] = strong

    # ---- search timing: product search vs the reference's search (CPU restatement)
    from oracle import search_port
    t_new, t_ref, t_a100 = [], [], []
    for (m, n, k) in README_SHAPES:
        cfg = MatmulConfig(m, n, k, 32)
        t0 = time.perf_counter(); get_roller_hints(cfg, arch, topk=20); t_new.append(time.perf_counter() - t0)
        t0 = time.perf_counter(); get_roller_hints(cfg, CUDA(), topk=20); t_a100.append(time.perf_counter() - t0)
        t0 = time.perf_counter(); search_port.roller_hints(m, n, k, topk=20); t_ref.append(time.perf_counter() - t0)
    roofline["search_ms"] = {"b200_policy": statistics.mean(t_new) * 1e3,
                             "a100_policy": statistics.mean(t_a100) * 1e3,
                             "reference_port": statistics.mean(t_ref) * 1e3}

    # ---- CPU baseline on this box's host cores (bounded sample)
    from oracle import gemm_oracle
    cpu_flops, cpu_secs, _, cpu_done = cpu_reference_pass(README_SHAPES, budget_s=15.0)
    cpu_baseline = {
        "value": cpu_flops / cpu_secs / 1e12, "unit": UNIT, "cores": gemm_oracle.host_threads(),
        "kind": "port",
        "sample": f"numpy fp32 matmul of the first {cpu_done} README shapes, one pass, all host threads",
        "search_ms_reference_port": statistics.mean(t_ref) * 1e3,
    }

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3 (fp32 in, fp32 accumulate/out)",
        "data": "synthetic",
        "config": workload_config(world),
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "path": ("roller_b200_gemm_host_async per shape, three streams" if world == 1 else
                         "mgpu.HostStagedGemm per shape: own rows of A and 1/world of B uploaded "
                         "per rank, B's shares exchanged over NVLink (bytes are per rank)"),
                "pcie_gbs": pcie,
                "pcie_bound_ms": e2e_bound_ms},
        "gpu_launches": len(README_SHAPES) * args.steps,
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
            "tiles": ["x".join(map(str, t[0])) + f"/cg{t[1]}" for t in tiles16],
        },
    }
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
    ap.add_argument("--parts", default="all,strong",
                    help="comma list; leave out 'strong' to skip the sharded jobs at N > 1; "
                         "'alljobs' also runs the 8-GPU jobs' code paths on fewer GPUs")
    ap.add_argument("--fused-shapes", default="",
                    help="sharded M13 job: also time the fused exchange with these rounds of the "
                         "progressive schedule, 'rounds:ratio,...' (ratio in percent)")
    ap.add_argument("--strong-budget-s", type=float, default=240.0,
                    help="seconds after which no further sharded job is started")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
