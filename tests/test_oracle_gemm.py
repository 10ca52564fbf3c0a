"""The CPU oracle of the GEMM: seeded inputs, exact product, reference-kernel restatement and
the arithmetic model of the tensor-core modes."""
from pathlib import Path

import numpy as np
import pytest

from oracle import gemm_oracle as g

GOLDEN = Path(__file__).resolve().parent / "golden" / "gemm_golden.npz"
CASES = {"tiny_uniform": "uniform", "ragged_normal": "normal", "ktail_uniform": "uniform",
         "positive": "positive"}


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_input_generator_is_pinned(golden):
    for name, dist in CASES.items():
        M, N, K, seed = (int(v) for v in golden[f"{name}/meta"])
        A, B = g.make_inputs(M, N, K, dist, seed)
        assert A.dtype == np.float32 and A.flags.c_contiguous
        assert np.array_equal(A, golden[f"{name}/A"]) and np.array_equal(B, golden[f"{name}/B"])
        assert np.array_equal(g.matmul_fp64(A, B), golden[f"{name}/C64"])


def test_reference_kernel_restatement_matches_exact_product(golden):
    # fp32 FMA accumulation in k order, as the reference's generated kernel does
    for name in CASES:
        A, B, C64 = golden[f"{name}/A"], golden[f"{name}/B"], golden[f"{name}/C64"]
        for rstep in (1, 32, 1000):
            C = g.sgemm_ref_c(A, B, rstep=rstep)
            assert g.err_norm(C, C64) < 2e-6, (name, rstep)
        # blocking the reduction does not change a sequential FMA chain
        assert np.array_equal(g.sgemm_ref_c(A, B, rstep=8), g.sgemm_ref_c(A, B, rstep=32))


def test_reference_kernel_accumulates_into_c(golden):
    A, B = golden["tiny_uniform/A"], golden["tiny_uniform/B"]
    once = g.sgemm_ref_c(A, B)
    twice = g.sgemm_ref_c(A, B, C=once.copy())
    assert np.allclose(twice, 2 * once, rtol=1e-6, atol=1e-6)


def test_numpy_fp32_is_within_cp_allclose_band(golden):
    for name in CASES:
        A, B, C64 = golden[f"{name}/A"], golden[f"{name}/B"], golden[f"{name}/C64"]
        assert g.err_norm(g.matmul_fp32(A, B), C64) < 2e-6


def test_split_is_exact_and_small():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-20, 20),
                        np.array([0.0, -0.0, 1.0, -1.0, 3.4e38, 1e-38, np.inf, -np.inf, np.nan],
                                 dtype=np.float32)])
    big, small = g.tf32_trunc(x), g.split_small(x)
    fin = np.isfinite(x)
    # both parts live on the 19-bit grid the tensor core reads
    assert np.all((big.view(np.uint32) & 0x1FFF) == 0)
    assert np.all((small[fin].view(np.uint32) & 0x1FFF) == 0)
    # big + small reproduces x to about 2^-21 relative
    # (away from the subnormal range, where the remainder itself runs out of bits)
    nrm = fin & (np.abs(x) > 1e-30)
    rel = np.abs((big[nrm].astype(np.float64) + small[nrm].astype(np.float64)) - x[nrm]) / np.abs(x[nrm])
    assert rel.max() <= 2.0 ** -21
    assert np.isnan(small[~fin]).all()  # inf - inf: infinities surface as nan in 3xTF32
    # C and numpy agree bit for bit
    for v in x[fin][:512]:
        c = np.float32(g._c().oracle_split_small(float(v)))
        assert c.view(np.uint32) == g.split_small(np.array([v], np.float32)).view(np.uint32)[0]


def test_mode_error_bands():
    # 1024-long reductions: the bands the GPU parity tests gate on
    for dist in ("uniform", "normal", "positive"):
        A, B = g.make_inputs(96, 80, 1024, dist, seed=11)
        C64 = g.matmul_fp64(A, B)
        e1 = g.err_norm(g.emulate_1xtf32(A, B), C64)
        e1t = g.err_norm(g.emulate_1xtf32(A, B, rounding="trunc"), C64)
        e3 = g.err_norm(g.emulate_3xtf32(A, B), C64)
        assert 1e-5 < e1 < e1t < 3e-3, (dist, e1, e1t)   # rounding beats truncation
        assert e3 < 5e-7, (dist, e3)
        ec = g.err_norm(g.gemm_3xtf32_c(A, B, chunk=128), C64)
        assert ec < 1e-6, (dist, ec)


def test_error_metrics():
    A, B = g.make_inputs(8, 8, 8, "uniform", 0)
    C64 = g.matmul_fp64(A, B)
    assert g.err_norm(C64, C64) == 0.0 and g.err_comp(C64, C64, A, B) == 0.0
    bumped = C64.copy()
    bumped[3, 4] += 1e-3
    assert abs(g.err_norm(bumped, C64) - 1e-3 / np.abs(C64).max()) < 1e-12


def test_edge_shapes():
    A, B = g.make_inputs(1, 1, 1, "uniform", 0)
    assert g.sgemm_ref_c(A, B).shape == (1, 1)
    A, B = g.make_inputs(3, 5, 7, "normal", 0)
    assert np.allclose(g.sgemm_ref_c(A, B), A @ B, atol=1e-5)
    assert np.allclose(g.gemm_3xtf32_c(A, B), A @ B, atol=1e-5)


# ------------------------------------------------------------------ 16-bit operands
GOLDEN16 = np.load(Path(__file__).resolve().parent / "golden" / "gemm16_golden.npz")
CASES16 = sorted({k.split("/")[0] for k in GOLDEN16.files})


def _values16(name):
    conv = g.from_bf16_bits if name.startswith("bf16") else g.from_f16_bits
    return conv(GOLDEN16[f"{name}/A"]), conv(GOLDEN16[f"{name}/B"])


@pytest.mark.parametrize("name", CASES16)
def test_golden16_is_reproduced_by_the_generator_and_the_model(name):
    M, N, K, seed = (int(v) for v in GOLDEN16[f"{name}/meta"])
    kind = "bf16" if name.startswith("bf16") else "f16"
    dist = {"bf16_uniform": "uniform", "bf16_ragged_normal": "normal", "f16_uniform": "uniform",
            "f16_ktail_positive": "positive"}[name]
    Ab, Bb, Av, Bv = g.make_inputs_16(M, N, K, kind, dist, seed)
    assert np.array_equal(Ab, GOLDEN16[f"{name}/A"]) and np.array_equal(Bb, GOLDEN16[f"{name}/B"])
    C64 = GOLDEN16[f"{name}/C64"]
    assert np.array_equal(g.matmul_fp64(Av, Bv), C64)
    # exact products + fp32 chunk sums: fp32-level error, far below the operands' own rounding
    assert g.err_norm(g.emulate_16bit(Av, Bv, chunk=64), C64) < 5e-7
    A32, B32 = g.make_inputs(M, N, K, dist, seed)
    rounding = g.err_norm(C64, g.matmul_fp64(A32, B32))
    assert (1e-4 if kind == "f16" else 1e-3) < rounding < (2e-3 if kind == "f16" else 2e-2)


def test_bf16_and_f16_conversions():
    x = np.array([0.0, -0.0, 1.0, 1.0 + 2.0**-8, 1.0 + 3 * 2.0**-8, 3.4028235e38, np.inf, -np.inf,
                  1e-40, 65504.0, 65520.0, 2.0**-25], dtype=np.float32)
    b = g.to_bf16_bits(x)
    # ties go to the even neighbour: 1 + 2^-8 -> 1.0, 1 + 3*2^-8 -> 1 + 2^-6
    assert list(g.from_bf16_bits(b)[:5]) == [0.0, 0.0, 1.0, 1.0, 1.0 + 2.0**-6]
    assert np.signbit(g.from_bf16_bits(b)[1])
    assert g.from_bf16_bits(b)[5] == np.inf            # rounds up past the largest bf16
    assert g.from_bf16_bits(b)[6] == np.inf and g.from_bf16_bits(b)[7] == -np.inf
    assert np.isnan(g.from_bf16_bits(g.to_bf16_bits(np.array([np.nan], np.float32)))[0])
    f = g.from_f16_bits(g.to_f16_bits(x))
    assert f[9] == 65504.0 and f[10] == np.inf and f[11] == 0.0
    with pytest.raises(ValueError):
        g.make_inputs_16(2, 2, 2, "fp8")


@pytest.mark.parametrize("name", CASES16)
def test_c_restatement_of_the_16_bit_arithmetic(name):
    kind = "bf16" if name.startswith("bf16") else "f16"
    Ab, Bb = GOLDEN16[f"{name}/A"], GOLDEN16[f"{name}/B"]
    Av, Bv = _values16(name)
    C64 = GOLDEN16[f"{name}/C64"]
    for chunk in (16, 64, 4096):
        Cc = g.gemm_16bit_c(Ab, Bb, kind, chunk=chunk)
        assert g.err_norm(Cc, C64) < 5e-7
        # same model as the numpy one (the fp64 partial sums may differ in their last bit)
        assert np.abs(Cc - g.emulate_16bit(Av, Bv, chunk=chunk)).max() <= 1e-6 * np.abs(C64).max()


def test_c_decoding_of_16_bit_patterns():
    """Every fp16 and a sweep of bf16 bit patterns through a 1 x 1 x 1 product with 1.0."""
    one16 = {"bf16": np.uint16(0x3F80), "f16": np.uint16(0x3C00)}
    for kind, conv in (("f16", g.from_f16_bits), ("bf16", g.from_bf16_bits)):
        pats = np.arange(0, 65536, 1 if kind == "f16" else 7, dtype=np.uint32).astype(np.uint16)
        A = pats.reshape(-1, 1)
        B = np.array([[one16[kind]]], dtype=np.uint16)
        with np.errstate(invalid="ignore"):
            got = g.gemm_16bit_c(A, B, kind)[:, 0]
        want = conv(pats)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok])
