"""Parity of the 16-bit-operand kernels (bf16 / fp16 A and B, fp32 accumulation and C), called
through the C ABI, with the CPU oracle.

Products of two 16-bit floats are exact in fp32, so against the fp64 product of the same rounded
operands the whole error is the accumulator's. Tolerance (max|C - C64| / max|C64|): <= 1e-5,
the bar of the fp32 path; measured 2.3e-6 with the default drain every 2048 k and ~5e-7 with
512 k, so the tests also hold the default to 5e-6.
"""
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mlir_roller_b200 import _lib, roller  # noqa: E402
from mlir_roller_b200.analyze import MODE_BF16, MODE_F16, MatmulConfig  # noqa: E402
from oracle import gemm_oracle as g  # noqa: E402

TOL = 1e-5
TIGHT = 5e-6
GOLDEN16 = np.load(Path(__file__).resolve().parent / "golden" / "gemm16_golden.npz")
TILES16 = [(256, 256, 2), (256, 128, 2), (128, 256, 1), (128, 128, 1), (128, 64, 1)]
SKINNY16 = [(64, 128, 1, 2), (32, 128, 1, 2)]
KINDS = {"bf16": (MODE_BF16, torch.bfloat16), "f16": (MODE_F16, torch.float16)}


def to_device(bits: np.ndarray, kind: str, ld: int | None = None):
    """uint16 bit patterns -> device tensor of the 16-bit float type, optionally with padded rows."""
    t = torch.from_numpy(bits.view(np.int16)).cuda().view(KINDS[kind][1])
    if ld is None or ld == t.shape[1]:
        return t.contiguous()
    out = torch.zeros(t.shape[0], ld, dtype=t.dtype, device="cuda")
    out[:, :t.shape[1]] = t
    return out


def gpu_gemm16(Ab, Bb, kind, tile, *, lda=None, ldb=None, ldc=None, flags=0, C0=None, chunk=None,
               stream_k=None, b_transposed=False):
    M, K = Ab.shape
    N = Bb.shape[1]
    ldc = N if ldc is None else ldc
    dA = to_device(Ab, kind, lda)
    if b_transposed:
        flags |= _lib.FLAG_B_TRANSPOSED
        dB = to_device(np.ascontiguousarray(Bb.T), kind, ldb)
    else:
        dB = to_device(Bb, kind, ldb)
    dC = torch.full((M, ldc), float("nan"), device="cuda")
    if C0 is not None:
        dC[:, :N] = torch.from_numpy(C0).cuda()
    plan = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, lda=dA.shape[1], ldb=dB.shape[1], ldc=ldc,
                         mode=KINDS[kind][0], flags=flags)
    if chunk is not None:
        plan.set_chunk(chunk)
    if stream_k is not None:
        plan.set_stream_k(stream_k)
    plan.run(dA, dB, dC)
    torch.cuda.synchronize()
    plan.check_status()
    out = dC.cpu().numpy()
    plan.destroy()
    if ldc > N:
        assert np.isnan(out[:, N:]).all()
    return out[:, :N]


@pytest.mark.parametrize("tile", TILES16 + SKINNY16)
@pytest.mark.parametrize("name", sorted({k.split("/")[0] for k in GOLDEN16.files}))
def test_golden_vectors(tile, name):
    kind = "bf16" if name.startswith("bf16") else "f16"
    C = gpu_gemm16(GOLDEN16[f"{name}/A"], GOLDEN16[f"{name}/B"], kind, tile)
    assert g.err_norm(C, GOLDEN16[f"{name}/C64"]) <= 1e-6


SHAPES = [(1, 1, 1), (7, 5, 3), (128, 256, 64), (129, 257, 65), (300, 200, 136), (512, 384, 1000),
          (1000, 1000, 2500), (64, 2048, 4096)]


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_against_oracle(shape, kind):
    """Ragged sizes in all three dimensions, odd leading dimensions included (rows that are not
    a multiple of 16 bytes go through the padded staging copy)."""
    M, N, K = shape
    Ab, Bb, Av, Bv = g.make_inputs_16(M, N, K, kind, "uniform", seed=M + N + K)
    C64 = g.matmul_fp64(Av, Bv)
    for tile in ((256, 256, 2), (128, 128, 1)):
        C = gpu_gemm16(Ab, Bb, kind, tile)
        assert g.err_norm(C, C64) <= TIGHT, (tile, g.err_norm(C, C64))
    # the arithmetic model (exact products, fp32 chunk sums) predicts the same band
    assert g.err_norm(g.emulate_16bit(Av, Bv), C64) <= TIGHT


def test_all_tiles_agree_bit_for_bit():
    """With whole-tile scheduling every tile reduces k in the same order: identical bits."""
    Ab, Bb, _, _ = g.make_inputs_16(512, 512, 1536, "bf16", "normal", seed=4)
    outs = [gpu_gemm16(Ab, Bb, "bf16", t, stream_k=0) for t in TILES16]
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    again = gpu_gemm16(Ab, Bb, "bf16", TILES16[0], stream_k=0)
    assert np.array_equal(again, outs[0])


def test_chunk_length_trades_accuracy():
    """Longer TMEM chunks = more truncating adds in a row: the error grows with the chunk."""
    Ab, Bb, Av, Bv = g.make_inputs_16(256, 256, 8192, "bf16", "uniform", seed=6)
    C64 = g.matmul_fp64(Av, Bv)
    # whole-tile schedule: a cut along K would shorten the chains by itself
    e = {c: g.err_norm(gpu_gemm16(Ab, Bb, "bf16", (256, 256, 2), chunk=c, stream_k=0), C64)
         for c in (256, 2048, 0)}
    assert e[256] < e[2048] < e[0]
    assert e[256] <= 1e-6 and e[2048] <= TIGHT and e[0] <= 5e-5


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_leading_dimensions_accumulate_and_transposed_b(kind):
    M, N, K = 200, 136, 264
    Ab, Bb, Av, Bv = g.make_inputs_16(M, N, K, kind, "normal", seed=8)
    C64 = g.matmul_fp64(Av, Bv)
    scale = np.abs(C64).max()
    C = gpu_gemm16(Ab, Bb, kind, (128, 128, 1), lda=K + 8, ldb=N + 16, ldc=N + 4)
    assert g.err_norm(C, C64) <= TIGHT
    C = gpu_gemm16(Ab, Bb, kind, (128, 128, 1), lda=K + 3, ldb=N + 5)      # staged copies
    assert g.err_norm(C, C64) <= TIGHT
    C0 = np.random.default_rng(1).standard_normal((M, N)).astype(np.float32)
    C = gpu_gemm16(Ab, Bb, kind, (256, 256, 2), flags=_lib.FLAG_ACCUMULATE, C0=C0)
    assert np.abs(C - (C64 + C0)).max() / scale <= TIGHT
    for tile in ((256, 256, 2), (128, 128, 1), (128, 64, 1)):
        C = gpu_gemm16(Ab, Bb, kind, tile, b_transposed=True)
        assert g.err_norm(C, C64) <= TIGHT


@pytest.mark.parametrize("tile", SKINNY16)
def test_skinny_layout(tile):
    for (M, N, K) in ((16, 1000, 520), (48, 512, 4096), (1, 128, 64)):
        Ab, Bb, Av, Bv = g.make_inputs_16(M, N, K, "bf16", "uniform", seed=N)
        C = gpu_gemm16(Ab, Bb, "bf16", tile)
        assert g.err_norm(C, g.matmul_fp64(Av, Bv)) <= TIGHT


def test_stream_k_schedule():
    """Leftover tiles cut along K give the same result within tolerance."""
    Ab, Bb, Av, Bv = g.make_inputs_16(2304, 2304, 4096, "bf16", "uniform", seed=9)  # 81 pair tiles
    C64 = g.sample_rows_fp64(Av, Bv, [0, 255, 256, 1151, 2303])
    for sk in (0, 1):
        C = gpu_gemm16(Ab, Bb, "bf16", (256, 256, 2), stream_k=sk, chunk=1024)
        assert g.err_norm(C[[0, 255, 256, 1151, 2303]], C64) <= TIGHT


def test_wrong_dtype_and_bad_arguments_are_rejected():
    tile = _lib.find_tile(128, 128, 1)
    plan = _lib.GemmPlan(tile, 64, 64, 64, mode=MODE_BF16)
    a32 = torch.zeros(64, 64, device="cuda")
    a16 = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        plan.run(a32, a16, a32)
    with pytest.raises(TypeError):
        plan.run(a16, a16.to(torch.float16), a32)
    with pytest.raises(TypeError):
        plan.run(a16, a16, a16)
    plan.destroy()
    with pytest.raises(_lib.RollerError):    # the 256x64 pair tile has no 16-bit kernel
        _lib.GemmPlan(_lib.find_tile(256, 64, 2), 64, 64, 64, mode=MODE_BF16)
    with pytest.raises(_lib.RollerError):
        _lib.GemmPlan(tile, 64, 64, 64, mode=18)


@pytest.mark.parametrize("mode", [MODE_BF16, MODE_F16])
def test_full_size_m13_sampled_rows(mode):
    """8192 x 4096 x 4096 through the search: sampled rows against the CPU fp64 product."""
    kind = "bf16" if mode == MODE_BF16 else "f16"
    M, N, K = 8192, 4096, 4096
    cfg = MatmulConfig(M, N, K, 16)
    hint, fn, _ = roller.best_hint(cfg, mode=mode, measure=False)
    assert hint.mode == mode and hint.rstep == 64
    gen = torch.Generator(device="cuda")
    gen.manual_seed(13)
    dt = KINDS[kind][1]
    A = (torch.rand(M, K, device="cuda", generator=gen) * 2 - 1).to(dt)
    B = (torch.rand(K, N, device="cuda", generator=gen) * 2 - 1).to(dt)
    C = torch.empty(M, N, device="cuda")
    fn.plan.run(A, B, C)
    torch.cuda.synchronize()
    fn.plan.check_status()
    rows = [0, 1, 127, 128, 255, 256, 4095, 4096, 8191]
    C64 = A[rows].double().cpu().numpy() @ B.double().cpu().numpy()
    assert g.err_norm(C[rows].cpu().numpy(), C64) <= TIGHT
    # and the whole matrix against the GPU's own fp64 product
    full = float((C.double() - A.double() @ B.double()).abs().max() / np.abs(C64).max())
    assert full <= TIGHT
    fn.plan.destroy()


def test_compiler_run_eval_and_baseline_for_a_16_bit_config(capsys):
    cfg = MatmulConfig(1024, 1024, 1024, 16)
    hint = roller.get_roller_hints(cfg, roller.B200(), topk=1)[0]
    fn = roller.Compiler(cfg, hint).compile()
    assert fn.plan.mode == MODE_BF16
    ms, gflops = roller.run_eval(fn, 2, hint, repeat_times=5)
    assert ms > 0 and gflops > 0
    ms_b, gflops_b = roller.run_baseline(cfg, repeat_times=5)
    assert ms_b > 0 and gflops_b > 0
    assert "differs" not in capsys.readouterr().out
    with pytest.raises(_lib.RollerError):
        roller.Compiler(cfg, hint, mode=3).compile()


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("tile", [(256, 256, 2), (128, 128, 1), (128, 64, 1), (32, 128, 1, 2)])
def test_c_in_the_operand_type(kind, tile):
    """FLAG_C_16BIT: the fp32 sums are rounded to nearest even once, on the store -- the result
    equals the fp32-C result converted by torch, bit for bit; ragged shapes, padded and odd
    leading dimensions and C += A@B included."""
    mode, dt = KINDS[kind]
    for (M, N, K, ldc) in ((300, 200, 136, 200), (256, 512, 192, 520), (70, 131, 64, 131)):
        Ab, Bb, _, _ = g.make_inputs_16(M, N, K, kind, "normal", seed=M)
        dA, dB = to_device(Ab, kind), to_device(Bb, kind)
        C32 = torch.empty(M, N, device="cuda")
        p32 = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, mode=mode)
        p32.run(dA, dB, C32)
        C16 = torch.full((M, ldc), 7.0, device="cuda", dtype=dt)
        p16 = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, ldc=ldc, mode=mode, flags=_lib.FLAG_C_16BIT)
        p16.run(dA, dB, C16)
        torch.cuda.synchronize()
        p16.check_status()
        assert torch.equal(C16[:, :N], C32.to(dt))
        assert (C16[:, N:] == 7.0).all()            # pad columns untouched
        # accumulate: old C is read in the 16-bit type, the sum is rounded once
        C0 = torch.randn(M, ldc, device="cuda").to(dt)
        Cacc = C0.clone()
        pacc = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, ldc=ldc, mode=mode,
                             flags=_lib.FLAG_C_16BIT | _lib.FLAG_ACCUMULATE)
        pacc.set_stream_k(0)
        p32.set_stream_k(0)
        p32.run(dA, dB, C32)
        pacc.run(dA, dB, Cacc)
        torch.cuda.synchronize()
        assert torch.equal(Cacc[:, :N], (C32 + C0[:, :N].float()).to(dt))
        with pytest.raises(TypeError):
            p16.run(dA, dB, C32)
        for p in (p32, p16, pacc):
            p.destroy()
    with pytest.raises(_lib.RollerError):           # fp32 operands have no 16-bit C
        _lib.GemmPlan(_lib.find_tile(128, 128, 1), 64, 64, 64, mode=3, flags=_lib.FLAG_C_16BIT)


def test_compiler_out_16bit():
    cfg = MatmulConfig(512, 768, 256, 16)
    hint = roller.get_roller_hints(cfg, roller.B200(), topk=1)[0]
    fn = roller.Compiler(cfg, hint, out_16bit=True).compile()
    A = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    B = torch.randn(256, 768, device="cuda").to(torch.bfloat16)
    C = torch.empty(512, 768, device="cuda", dtype=torch.bfloat16)
    fn.plan.run(A, B, C)
    torch.cuda.synchronize()
    ref = (A.double() @ B.double())
    assert float((C.double() - ref).abs().max() / ref.abs().max()) < 8e-3   # bf16 output rounding


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_special_values(kind):
    """IEEE behaviour of the 16-bit path: inf and nan propagate, inf * 0 along a row is nan,
    a sum beyond the fp32 range would need > 3e38 (not reachable here), fp16 subnormal inputs
    are exact, and a 16-bit C overflows to inf where the fp32 C holds a finite value."""
    A = np.zeros((128, 64), np.float32)
    B = np.zeros((64, 64), np.float32)
    A[0, 0] = np.inf; B[0, 0] = 1.0
    A[1, 1] = 2.0 ** -20; B[1, 1] = 2.0 ** -4            # fp16: subnormal times normal, exact
    A[2, 2] = 300.0; B[2, 2] = 300.0                     # 9e4: beyond fp16's 65504 as an output
    A[3, 3] = np.nan; B[3, 3] = 2.0
    conv = g.to_bf16_bits if kind == "bf16" else g.to_f16_bits
    Ab, Bb = conv(A), conv(B)
    C = gpu_gemm16(Ab, Bb, kind, (128, 64, 1))
    assert np.isinf(C[0, 0]) and C[0, 0] > 0
    assert np.isnan(C[0, 1]) and np.isnan(C[3, 3])
    assert C[1, 1] == np.float32(2.0 ** -24) and C[2, 2] == 90000.0
    mode, dt = KINDS[kind]
    plan = _lib.GemmPlan(_lib.find_tile(128, 64, 1), 128, 64, 64, mode=mode, flags=_lib.FLAG_C_16BIT)
    C16 = torch.empty(128, 64, device="cuda", dtype=dt)
    plan.run(to_device(Ab, kind), to_device(Bb, kind), C16)
    torch.cuda.synchronize()
    plan.destroy()
    out = C16.float().cpu().numpy()
    assert np.isinf(out[0, 0]) and np.isnan(out[3, 3])
    assert (np.isinf(out[2, 2]) if kind == "f16" else out[2, 2] == 90112.0)   # bf16: nearest value
