"""Generates tests/golden/gemm16_golden.npz: small seeded GEMM cases with 16-bit operands.

    python tests/golden/gen_gemm16_golden.py

The reference's problem descriptor carries the element width (el_bits, src/analyze.py:31,39-41)
but its kernel generator only emits f32 (src/roller.py:47-68), so there is nothing of the
reference to record for 16-bit operands; like gemm_golden.npz these vectors come from the
definition. Operands are the seeded fp32 inputs of the other fixture rounded to bf16 / fp16
(round to nearest even) and stored as bit patterns, so what the device receives is pinned
exactly; the product of the rounded values is computed in float64.
"""
from pathlib import Path
import sys

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from oracle import gemm_oracle  # noqa: E402

CASES = [  # name, kind, M, N, K, dist, seed
    ("bf16_uniform", "bf16", 40, 72, 136, "uniform", 10),
    ("bf16_ragged_normal", "bf16", 70, 50, 97, "normal", 11),
    ("f16_uniform", "f16", 40, 72, 136, "uniform", 12),
    ("f16_ktail_positive", "f16", 48, 64, 45, "positive", 13),
]


def main() -> None:
    out = {}
    for name, kind, M, N, K, dist, seed in CASES:
        Ab, Bb, Av, Bv = gemm_oracle.make_inputs_16(M, N, K, kind, dist, seed)
        out[f"{name}/A"] = Ab
        out[f"{name}/B"] = Bb
        out[f"{name}/C64"] = gemm_oracle.matmul_fp64(Av, Bv)
        out[f"{name}/meta"] = np.array([M, N, K, seed])
    dst = Path(__file__).resolve().parent / "gemm16_golden.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
