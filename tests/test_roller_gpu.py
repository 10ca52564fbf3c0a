"""The drop-in Python surface (Compiler / run_eval / run_baseline / benchmark / mgpu) on a GPU."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mlir_roller_b200 import B200, CUDA, MatmulConfig, _lib, get_roller_hints, mgpu, roller  # noqa: E402
from mlir_roller_b200 import benchmark as bm  # noqa: E402
from oracle import gemm_oracle as g  # noqa: E402


def test_compile_and_call_like_the_reference():
    cfg = MatmulConfig(512, 384, 256, 32)
    hint = get_roller_hints(cfg, B200(), topk=1)[0]
    fn = roller.Compiler(cfg, hint, pipeline_depth=2, dump_path=None).compile()
    A, B = g.make_inputs(512, 384, 256, "uniform", 0)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.zeros(512, 384, device="cuda")
    grid = (384 // hint.block_tile[1] or 1, 512 // hint.block_tile[0] or 1)
    fn(grid, (8, 16), (dA.data_ptr(), dB.data_ptr(), dC.data_ptr()), shared_mem=hint.smem_cost * 2)
    torch.cuda.synchronize()
    assert g.err_norm(dC.cpu().numpy(), g.matmul_fp64(A, B)) <= 1e-5
    info = fn.launch_info()
    assert info["block"] == 512 and info["smem_bytes"] <= 227 * 1024
    with pytest.raises(ValueError):
        fn((0, 1), (1, 1), (dA.data_ptr(), dB.data_ptr(), dC.data_ptr()))


def test_reference_policy_hints_bind_when_a_kernel_exists():
    cfg = MatmulConfig(1024, 1024, 512, 32)
    hints = get_roller_hints(cfg, CUDA(), topk=20)
    bound, skipped = 0, 0
    for h in hints:
        try:
            roller.Compiler(cfg, h).compile()
            bound += 1
        except _lib.RollerError as e:
            assert e.status == _lib.ERR_UNSUPPORTED
            skipped += 1
    assert bound >= 1 and skipped >= 1  # [128,128] binds; e.g. [64,64] has no sm_100a kernel


def test_run_eval_and_baseline(capsys):
    cfg = MatmulConfig(1024, 1024, 1024, 32)
    hint = get_roller_hints(cfg, B200(), topk=1)[0]
    fn = roller.Compiler(cfg, hint).compile()
    ms, gflops = roller.run_eval(fn, 2, hint, repeat_times=5)
    assert ms > 0 and abs(gflops - 2 * 1024 ** 3 * 1e-9 / (ms / 1e3)) / gflops < 1e-6
    bms, bg = roller.run_baseline(cfg, repeat_times=5)
    assert bms > 0 and bg > 0
    out = capsys.readouterr().out
    assert "GFLOPS=" in out and "differs" not in out  # passes the reference's allclose check


def test_best_hint_measures():
    cfg = MatmulConfig(1024, 2048, 512, 32)
    hint, fn, ms = roller.best_hint(cfg, B200(), topk=3)
    assert ms > 0 and hint.block_tile[0] in (128, 256)


def test_benchmark_sweep_writes_csv(tmp_path):
    csv = tmp_path / "benchmark_results.csv"
    df = bm.benchmark([(512, 512, 512), (300, 200, 100)], topk=2, csv_path=str(csv))
    assert csv.exists() and len(df) == 2
    for col in ["M", "N", "K", "CuPy Time (ms)", "CuPy GFLOPS", "Roller Time (ms)", "Roller GFLOPS",
                "Speedup vs CuPy", "Best Hint"]:
        assert col in df.columns
    assert (df["max_rel_err"] <= 1e-5).all()


def test_sharded_gemm_on_one_gpu_emulating_ranks():
    # ranks are emulated one after another on this GPU; the gather itself is covered by the
    # gloo test on CPU
    M, N, K = 1024, 768, 640
    A, B = g.make_inputs(M, N, K, "uniform", seed=13)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    C64 = g.matmul_fp64(A, B)
    for world, grid in ((2, (2, 1)), (4, (2, 2)), (8, (4, 2))):
        full = torch.full((M, N), float("nan"), device="cuda")
        for rank in range(world):
            sg = mgpu.ShardedGemm(M, N, K, rank, world, grid=grid)
            b = sg.block
            a_rows, _ = sg.local_operands(dA, dB)
            c_blk = torch.empty(b.rows, b.cols, device="cuda")
            sg.run(a_rows.contiguous(), dB, c_blk)
            full[b.row0:b.row1, b.col0:b.col1] = c_blk
        torch.cuda.synchronize()
        assert g.err_norm(full.cpu().numpy(), C64) <= 1e-5, grid


def test_best_hint_uses_and_fills_the_cache(tmp_path):
    cfg = MatmulConfig(768, 1024, 512, 32)
    cache = roller.TuneCache(tmp_path / "tune.json", device_name=_lib.device_info(0).name.decode())
    hint, fn, ms = roller.best_hint(cfg, B200(), topk=3, cache=cache)
    assert cache.get(cfg, 3)[:3] == (hint.block_tile[0], hint.block_tile[1], hint.cta_group)
    hint2, fn2, ms2 = roller.best_hint(cfg, B200(), topk=3, measure=False,
                                       cache=roller.TuneCache(tmp_path / "tune.json",
                                                              device_name=cache.device_name))
    assert hint2.block_tile == hint.block_tile and ms2 == ms


def test_calibrate_measures_per_kblock_times():
    """The device model's per-k-block table can be re-measured on the GPU at hand; the figures
    land near the shipped table and the ranking of a large square problem is unchanged."""
    from mlir_roller_b200 import arch as arch_mod
    shipped = arch_mod.B200()
    model = roller.calibrate(iters=3, k_short=1024, k_long=4096)
    for key, (t1, t3) in model.kblock_us.items():
        s1, s3 = shipped.kblock_us[key]
        assert 0.5 * s1 < t1 < 2.0 * s1, (key, t1, s1)
        assert 0.5 * s3 < t3 < 2.0 * s3, (key, t3, s3)
    for key, t in model.kblock_us_16.items():
        assert 0.5 * shipped.kblock_us_16[key] < t < 2.0 * shipped.kblock_us_16[key], (key, t)
    for mode in (1, 3):
        top = roller.get_roller_hints(roller.MatmulConfig(8192, 8192, 8192, 32), model, topk=1, mode=mode)[0]
        assert (top.block_tile, top.cta_group) == ([256, 256], 2)


def test_cut_along_k_pays_on_an_underfilled_grid():
    """4096 x 64 x 8192 in 1xTF32: 32 tiles for 148 SMs. By default the library deals the
    tiles out along K; the result stays within the 1xTF32 band and the launch is faster than
    with whole tiles."""
    M, N, K = 4096, 64, 8192
    cfg = MatmulConfig(M, N, K, 32)
    hint = get_roller_hints(cfg, B200(), topk=1, mode=1)[0]
    A, Bm = g.make_inputs(M, N, K, "uniform", seed=3)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(Bm).cuda()
    dC = torch.empty(M, N, device="cuda")
    split = roller.Compiler(cfg, hint, mode=1).compile()
    whole = roller.Compiler(cfg, hint, mode=1, stream_k=0).compile()
    split((1, 1), (1, 1), (dA.data_ptr(), dB.data_ptr(), dC.data_ptr()))
    torch.cuda.synchronize()
    split.plan.check_status()
    rows = [0, 127, 128, 2047, 4095]
    assert g.err_norm(dC.cpu().numpy()[rows], g.sample_rows_fp64(A, Bm, rows)) <= 2e-3
    # Measured on an idle B200: 35 us against 76 us. The GPU is shared and power-capped, so only
    # the direction is asserted, on the best of several repeats.
    t_split = min(split.time(dA, dB, dC, warmup=3, iters=20) for _ in range(5))
    t_whole = min(whole.time(dA, dB, dC, warmup=3, iters=20) for _ in range(5))
    print(f"cut along K: {t_split * 1e3:.1f} us, whole tiles: {t_whole * 1e3:.1f} us")
    assert t_split < t_whole, (t_split, t_whole)
