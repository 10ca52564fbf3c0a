"""Generates tests/golden/gemm_golden.npz: small seeded GEMM cases with their exact products.

    python tests/golden/gen_gemm_golden.py

The reference holds no golden outputs for its kernel (its only check, src/roller.py:552-554,
prints on mismatch), so these vectors are produced from the definition: operands from
numpy.random.default_rng(seed) (A drawn before B), product in float64. They pin (a) the input
generator used by every parity test and (b) the expected result for the GPU parity tests, so a
change in either shows up as a diff of this file.
"""
from pathlib import Path
import sys

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from oracle import gemm_oracle  # noqa: E402

CASES = [  # name, M, N, K, dist, seed
    ("tiny_uniform", 24, 40, 56, "uniform", 0),
    ("ragged_normal", 130, 70, 97, "normal", 1),
    ("ktail_uniform", 64, 96, 45, "uniform", 2),
    ("positive", 96, 64, 128, "positive", 3),
]


def main() -> None:
    out = {}
    for name, M, N, K, dist, seed in CASES:
        A, B = gemm_oracle.make_inputs(M, N, K, dist, seed)
        out[f"{name}/A"] = A
        out[f"{name}/B"] = B
        out[f"{name}/C64"] = gemm_oracle.matmul_fp64(A, B)
        out[f"{name}/meta"] = np.array([M, N, K, seed])
    dst = Path(__file__).resolve().parent / "gemm_golden.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
