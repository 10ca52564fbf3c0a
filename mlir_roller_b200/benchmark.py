"""Sweep harness: per shape, time the library baseline, search rTile hints, time every hint and
keep the fastest; print a table and write `benchmark_results.csv`.

Same entry point and CSV columns as the reference's src/benchmark.py:10-95 (the "CuPy" columns
hold the cuBLAS baseline, here reached through torch), plus columns the B200 build adds: search
time, arithmetic mode, TFLOPS, fraction of the tensor roofline and the error against fp64.
"""
from __future__ import annotations

import itertools
import time
from pathlib import Path

import pandas as pd

from .analyze import MODE_3XTF32, MatmulConfig, get_roller_hints
from .arch import B200
from .roller import Compiler, run_baseline, run_eval

# The 14 shapes of the reference's published table (README.md:12-17), M0..M13.
README_SHAPES = [
    (2048, 2048, 2048), (2048, 2048, 8192), (2048, 4096, 2048), (2048, 4096, 4096),
    (2048, 8192, 2048), (2048, 8192, 4096), (2048, 8192, 8192), (4096, 2048, 2048),
    (4096, 4096, 8192), (4096, 8192, 2048), (4096, 8192, 4096), (8192, 2048, 8192),
    (8192, 4096, 2048), (8192, 4096, 4096),
]


def _error_vs_fp64(cuda_func, config: MatmulConfig, seed: int = 0) -> float:
    """max |C - C64| / max |C64| on seeded U[-1,1) inputs, fp64 product computed on the GPU."""
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    from .roller import operand_dtype
    dt = operand_dtype(cuda_func.plan.mode)     # 16-bit kernels: fp64 product of the rounded inputs
    A = (torch.rand(config.M, config.K, device="cuda", generator=g) * 2 - 1).to(dt)
    B = (torch.rand(config.K, config.N, device="cuda", generator=g) * 2 - 1).to(dt)
    C = torch.empty(config.M, config.N, device="cuda")
    cuda_func((1, 1), (1, 1), (A.data_ptr(), B.data_ptr(), C.data_ptr()))
    C64 = A.double() @ B.double()
    return float((C.double() - C64).abs().max() / C64.abs().max())


def benchmark(test_shapes: list[tuple[int, int, int]], topk: int = 20, mode: int = MODE_3XTF32,
              arch=None, csv_path: str = "benchmark_results.csv", check_error: bool = True):
    arch = B200() if arch is None else arch
    results = []
    for m, n, k in test_shapes:
        print(f"--- Benchmarking M={m}, N={n}, K={k} ---")
        sixteen = mode in (16, 17)
        config = MatmulConfig(M=m, N=n, K=k, el_bits=16 if sixteen else 32)

        print("Running baseline (cuBLAS via torch, same operand type)...")
        try:
            baseline_time, baseline_gflops = run_baseline(config, mode=mode)
            print(f"cuBLAS baseline: {baseline_time:.6f} ms, {baseline_gflops:.6f} GFLOPS")
        except Exception as e:  # noqa: BLE001 - mirror the reference: report and go on
            print(f"cuBLAS baseline failed: {e}")
            baseline_time, baseline_gflops = float("inf"), 0

        pipeline_depth = 2
        print(f"Generating and testing {topk} roller hints...")
        t0 = time.perf_counter()
        try:
            hints = get_roller_hints(config, arch, topk=topk, mode=mode)
        except Exception as e:  # noqa: BLE001
            print(f"Could not get hints for shape ({m},{n},{k}): {e}")
            hints = []
        search_ms = (time.perf_counter() - t0) * 1e3

        best_time, best_gflops, best_hint, best_func = float("inf"), 0, None, None
        for i, hint in enumerate(hints):
            print(f"  Testing hint {i + 1}/{len(hints)}: {hint}")
            try:
                cuda_func = Compiler(config, hint, pipeline_depth, dump_path=Path("log"),
                                     mode=mode).compile()
                t, gflops = run_eval(cuda_func, pipeline_depth, hint)
                if t < best_time:
                    best_time, best_gflops, best_hint, best_func = t, gflops, hint, cuda_func
            except Exception as e:  # noqa: BLE001 - a hint without a kernel is skipped
                print(f"    Hint failed with error: {e}")
                continue

        if best_hint:
            print(f"Best roller kernel: {best_time:.6f} ms, {best_gflops:.6f} GFLOPS")
            print(f"Best hint: {best_hint}")
        else:
            print("All roller hints failed.")

        err = _error_vs_fp64(best_func, config) if (best_func and check_error) else float("nan")
        tensor_tflops = best_gflops * (1 if sixteen else mode) / 1e3
        peak = getattr(arch, "bf16_tflops" if sixteen else "tf32_tflops", float("nan"))
        results.append({
            "M": m, "N": n, "K": k,
            "CuPy Time (ms)": baseline_time,
            "CuPy GFLOPS": baseline_gflops,
            "Roller Time (ms)": best_time,
            "Roller GFLOPS": best_gflops,
            "Speedup vs CuPy": (baseline_time / best_time
                                if best_time > 0 and baseline_time != float("inf") else 0),
            "Best Hint": str(best_hint) if best_hint else "N/A",
            "search_ms": search_ms,
            "mode": {16: "bf16", 17: "fp16"}.get(mode, f"{mode}xTF32"),
            "tflops": best_gflops / 1e3,
            "roofline_frac": tensor_tflops / peak,
            "max_rel_err": err,
        })
        # keep partial results if the sweep is interrupted
        pd.DataFrame(results).to_csv(csv_path, index=False)
        print("-" * 50)

    df = pd.DataFrame(results)
    print("\n--- Benchmark Summary ---")
    print(df.to_string())
    df.to_csv(csv_path, index=False)
    print(f"\nResults saved to {csv_path}")
    return df


if __name__ == "__main__":
    dims = [2048, 4096, 8192]
    benchmark(list(itertools.product(dims, dims, dims)))
