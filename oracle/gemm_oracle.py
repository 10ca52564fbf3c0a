"""TEST INFRASTRUCTURE -- CPU oracle for the fp32 GEMM of the Roller hot path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
module; the product (mlir_roller_b200/) never does.

What it restates
  * the result the reference checks its kernel against: an fp32 product of the same operands
    (`cp.allclose(dC, dA @ dB)`, src/roller.py:552-554) -- here `matmul_fp32` (numpy/BLAS) --
    and the exact product in fp64 that both are judged by (`matmul_fp64`);
  * the semantics of the generated `gemm_kernel`: C += A @ B on a host-zeroed C, fp32
    multiply-add in k order, k blocked by the hint's reduce step (src/roller.py:47-68,534);
    `sgemm_ref.c` next to this file is the plain-C form used for small cases;
  * the arithmetic model of the B200 kernels (split of an fp32 word into the 19 bits the tensor
    core reads plus a rounded remainder; 1 or 3 products per element) so that tests can predict
    the error band of each mode.

Parity status: PARITY UNPINNED for the GEMM arithmetic. The reference holds no golden vectors or
asserting tests for its kernel's output (its only check prints on mismatch and carries on), and
its GPU path (IREE fork + CuPy) cannot run here, so this oracle is anchored on the definition
(fp64 product of the same seeded inputs), not on reference outputs.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


# ------------------------------------------------------------------ seeded inputs
def make_inputs(M: int, N: int, K: int, dist: str = "uniform", seed: int = 0):
    """A (M,K) then B (K,N), row-major fp32, from one `default_rng(seed)` stream.

    dist: "uniform" = U[-1,1) (the benchmark configurations), "normal" = N(0,1) (the ragged /
    skinny configurations), "positive" = U[0,1) (what the reference's run_eval draws,
    src/roller.py:532-533).
    """
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        A = rng.uniform(-1.0, 1.0, (M, K)).astype(np.float32)
        B = rng.uniform(-1.0, 1.0, (K, N)).astype(np.float32)
    elif dist == "normal":
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = rng.standard_normal((K, N)).astype(np.float32)
    elif dist == "positive":
        A = rng.uniform(0.0, 1.0, (M, K)).astype(np.float32)
        B = rng.uniform(0.0, 1.0, (K, N)).astype(np.float32)
    else:
        raise ValueError(dist)
    return A, B


# ------------------------------------------------------------------ products
def matmul_fp64(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    return A.astype(np.float64) @ B.astype(np.float64)


def matmul_fp32(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """fp32 product with the host BLAS: the CPU stand-in for the reference's fp32 matmul."""
    return A.astype(np.float32, copy=False) @ B.astype(np.float32, copy=False)


def sample_rows_fp64(A: np.ndarray, B: np.ndarray, rows) -> np.ndarray:
    """Exact rows of the product, for shapes too large for a full fp64 product."""
    return A[np.asarray(rows)].astype(np.float64) @ B.astype(np.float64)


# ------------------------------------------------------------------ error metrics
def err_norm(C: np.ndarray, C64: np.ndarray) -> float:
    """max |C - C64| / max |C64|: the gate (1e-5 for 3xTF32). Element-wise relative error is
    not used: with sign-mixed inputs even a correctly rounded fp32 product has elements whose
    relative error is large."""
    return float(np.max(np.abs(C.astype(np.float64) - C64)) / np.max(np.abs(C64)))


def err_comp(C: np.ndarray, C64: np.ndarray, A: np.ndarray, B: np.ndarray) -> float:
    """max |C - C64| / (|A| |B|): component-wise backward-error style figure."""
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    return float(np.max(np.abs(C.astype(np.float64) - C64) / np.maximum(bound, 1e-300)))


# ------------------------------------------------------------------ tensor-core arithmetic model
def tf32_trunc(x: np.ndarray) -> np.ndarray:
    """The 19 bits (sign, 8 exponent, 10 mantissa) the tensor core reads of an fp32 word."""
    return (x.astype(np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def split_small(x: np.ndarray) -> np.ndarray:
    """What the split warps store: x - trunc19(x), exact in fp32, then rounded to the 19-bit
    grid by adding half a unit before the hardware truncation; nan for inf/nan (inf - inf)."""
    x = x.astype(np.float32)
    with np.errstate(invalid="ignore"):
        small = (x - tf32_trunc(x)).astype(np.float32)
    bits = (small.view(np.uint32) + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return bits.view(np.float32)


def tf32_round(x: np.ndarray) -> np.ndarray:
    """fp32 rounded to the nearest TF32 value (ties away from zero): what the TMA unit delivers
    for a tensor map of TFLOAT32 type, which is how the 1xTF32 kernels load their operands."""
    bits = x.astype(np.float32).view(np.uint32)
    return ((bits + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


def emulate_1xtf32(A: np.ndarray, B: np.ndarray, rounding: str = "nearest") -> np.ndarray:
    """1xTF32 with an ideal (fp64) accumulator: isolates the error of the 10-bit-mantissa
    inputs. "nearest" models the kernels (operands rounded on load), "trunc" what the tensor
    core does with raw fp32 words."""
    cut = tf32_round if rounding == "nearest" else tf32_trunc
    return cut(A).astype(np.float64) @ cut(B).astype(np.float64)


def emulate_3xtf32(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """3xTF32 with an ideal accumulator: small*big + big*small + big*big."""
    Ab, Bb = tf32_trunc(A).astype(np.float64), tf32_trunc(B).astype(np.float64)
    As, Bs = split_small(A).astype(np.float64), split_small(B).astype(np.float64)
    return As @ Bb + Ab @ Bs + Ab @ Bb


# ------------------------------------------------------------------ 16-bit operands
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even; nan stays nan."""
    bits = x.astype(np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    nan = np.isnan(x.astype(np.float32))
    return np.where(nan, np.uint32(0x7FC0), rounded).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    """bf16 bit patterns -> the fp32 values they denote (exact)."""
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> fp16 bit patterns (uint16), round to nearest even (numpy's conversion)."""
    return x.astype(np.float32).astype(np.float16).view(np.uint16)


def from_f16_bits(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def make_inputs_16(M: int, N: int, K: int, kind: str, dist: str = "uniform", seed: int = 0):
    """Seeded operands of `make_inputs`, rounded to bf16 or fp16: returns the bit patterns
    (uint16, what the device receives) and the fp32 values they denote."""
    A, B = make_inputs(M, N, K, dist, seed)
    if kind == "bf16":
        Ab, Bb = to_bf16_bits(A), to_bf16_bits(B)
        return Ab, Bb, from_bf16_bits(Ab), from_bf16_bits(Bb)
    if kind == "f16":
        Ab, Bb = to_f16_bits(A), to_f16_bits(B)
        return Ab, Bb, from_f16_bits(Ab), from_f16_bits(Bb)
    raise ValueError(f"kind must be 'bf16' or 'f16', not {kind!r}")


def emulate_16bit(Av: np.ndarray, Bv: np.ndarray, chunk: int = 2048) -> np.ndarray:
    """Model of the 16-bit kernels' arithmetic on the VALUES of the rounded operands: products
    of two 16-bit floats are exact in fp32; within a chunk of the reduction the accumulator is
    modelled as ideal (fp64), each chunk result is rounded to fp32 and the chunk results are
    added in fp32 with round-to-nearest, as the accumulate warps do."""
    K = Av.shape[1]
    out = np.zeros((Av.shape[0], Bv.shape[1]), dtype=np.float32)
    for k0 in range(0, K, chunk):
        part = Av[:, k0:k0 + chunk].astype(np.float64) @ Bv[k0:k0 + chunk].astype(np.float64)
        out = (out + part.astype(np.float32)).astype(np.float32)
    return out


# ------------------------------------------------------------------ plain-C restatement
_clib = None


def build_c(force: bool = False) -> Path:
    """Compile sgemm_ref.c into oracle/liboracle_sgemm.so with gcc."""
    import subprocess
    src, dst = HERE / "sgemm_ref.c", HERE / "liboracle_sgemm.so"
    if force or not dst.exists() or dst.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", str(dst),
                        str(src), "-lm"], check=True)
    return dst


def _c():
    global _clib
    if _clib is None:
        lib = ctypes.CDLL(str(build_c()))
        f32p = ctypes.POINTER(ctypes.c_float)
        lib.oracle_sgemm_accumulate.argtypes = [f32p, f32p, f32p] + [ctypes.c_int] * 4
        lib.oracle_sgemm_accumulate.restype = None
        lib.oracle_gemm_3xtf32.argtypes = [f32p, f32p, f32p] + [ctypes.c_int] * 4
        lib.oracle_gemm_3xtf32.restype = None
        lib.oracle_split_small.argtypes = [ctypes.c_float]
        lib.oracle_split_small.restype = ctypes.c_float
        _clib = lib
    return _clib


def _ptr(x: np.ndarray):
    return x.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def sgemm_ref_c(A: np.ndarray, B: np.ndarray, C: np.ndarray | None = None, rstep: int = 32):
    """C += A @ B the way the reference's generated kernel does it (fp32 FMA, k ascending in
    blocks of `rstep`); small sizes only. Returns the updated C."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    M, K = A.shape
    N = B.shape[1]
    C = np.zeros((M, N), np.float32) if C is None else np.ascontiguousarray(C, dtype=np.float32)
    _c().oracle_sgemm_accumulate(_ptr(A), _ptr(B), _ptr(C), M, N, K, rstep)
    return C


def gemm_3xtf32_c(A: np.ndarray, B: np.ndarray, chunk: int = 128) -> np.ndarray:
    """Plain-C model of the 3xTF32 kernel: split operands, products accumulated per `chunk` of k
    in double (standing in for the TMEM accumulator), chunks summed in fp32 round-to-nearest."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    M, K = A.shape
    N = B.shape[1]
    C = np.zeros((M, N), np.float32)
    _c().oracle_gemm_3xtf32(_ptr(A), _ptr(B), _ptr(C), M, N, K, chunk)
    return C


def gemm_16bit_c(Ab: np.ndarray, Bb: np.ndarray, kind: str, chunk: int = 2048) -> np.ndarray:
    """The C restatement of the 16-bit kernels' arithmetic on bf16 / fp16 bit patterns."""
    lib = _c()
    Ab = np.ascontiguousarray(Ab, dtype=np.uint16)
    Bb = np.ascontiguousarray(Bb, dtype=np.uint16)
    M, K = Ab.shape
    N = Bb.shape[1]
    C = np.empty((M, N), dtype=np.float32)
    lib.oracle_gemm_16bit(_ptr(Ab), _ptr(Bb), _ptr(C), M, N, K, {"bf16": 0, "f16": 1}[kind], chunk)
    return C


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
