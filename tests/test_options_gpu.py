"""Run-time options of a plan (roller_b200_gemm_set_option), called through the C ABI:
the TMA-store output path, the progressive schedule, launches that overlap the previous
kernel's tail, the limit of the device-side waits -- including one wait that really runs out --
and the arrival flags of the multi-GPU exchange.

Nothing here faults or hangs the GPU: the one failure that is provoked is a bounded wait on a
flag that is never raised, with a limit of about a millisecond, after which the kernel winds
down by itself and the host reads an error code.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from mlir_roller_b200 import _lib  # noqa: E402
from oracle import gemm_oracle as g  # noqa: E402

TOL_3X = 1e-5
TIGHT_3X = 4e-6
TOL_1X = 2e-3
# rTiles whose 3xTF32 kernel has the staging area of the TMA-store path
STAGED_3X = [(256, 256, 2), (256, 128, 2), (128, 256, 1), (128, 128, 1), (128, 64, 1)]


def run_plan(A, B, tile, mode, options=(), ldc=None, stream_k=None, launches=1, info=None):
    M, K = A.shape
    N = B.shape[1]
    ldc = N if ldc is None else ldc
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, ldc), float("nan"), device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, ldc=ldc, mode=mode)
    if stream_k is not None:
        plan.set_stream_k(stream_k)
    for opt, val in options:
        plan.set_option(opt, val)
    if info is not None:
        info.update(plan.launch_info())
        info.update(plan.schedule_info())
    outs = []
    for _ in range(launches):
        dC.fill_(float("nan"))
        plan.run(dA, dB, dC)
        torch.cuda.synchronize()
        plan.check_status()
        outs.append(dC.cpu().numpy())
    plan.destroy()
    for out in outs:
        if ldc > N:
            assert np.isnan(out[:, N:]).all()      # the pad columns of C are never written
    return [o[:, :N] for o in outs]


@pytest.mark.parametrize("tile", STAGED_3X)
@pytest.mark.parametrize("shape", [(512, 512, 256), (300, 200, 100), (1111, 776, 555), (129, 260, 33)])
def test_tma_store_writes_the_same_c(tile, shape):
    """C through shared memory and TMA stores is bit-identical to C stored by the accumulate
    warps, tails included (the TMA unit clips a box at the edge of the matrix), and nothing
    lands in the pad columns of a wide C."""
    M, N, K = shape
    A, B = g.make_inputs(M, N, K, "uniform", seed=M + K)
    for ldc in (N, N + 8):
        plain = run_plan(A, B, tile, 3, [(_lib.OPT_TMA_STORE, 0)], stream_k=0, ldc=ldc)[0]
        staged = run_plan(A, B, tile, 3, [(_lib.OPT_TMA_STORE, 1)], stream_k=0, ldc=ldc, launches=2)
        assert not np.isnan(staged[0]).any()
        assert np.array_equal(staged[0], plain) and np.array_equal(staged[1], plain)
    assert g.err_norm(plain, g.matmul_fp64(A, B)) <= TIGHT_3X


def test_the_shorter_ring_form_of_a_kernel_gives_the_same_bits():
    """The 1xTF32 and bf16 kernels of the 256 x 256 pair tile fill shared memory with their
    ring; a second form of each has one stage less and the staging area of the TMA-store path.
    The library binds that form by itself up to K = 4096 and the deeper ring beyond; both give
    the same C, as does the deeper ring told to use TMA stores (which switches forms)."""
    tile = _lib.find_tile(256, 256, 2)
    for K in (1024, 4352):
        M, N = 512, 768
        A, B = g.make_inputs(M, N, K, "uniform", seed=K)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        outs = []
        for option in (None, 0, 1):
            plan = _lib.GemmPlan(tile, M, N, K, mode=1)
            plan.set_stream_k(0)
            if option is not None:
                plan.set_option(_lib.OPT_TMA_STORE, option)
            dC = torch.full((M, N), float("nan"), device="cuda")
            plan.run(dA, dB, dC)
            torch.cuda.synchronize()
            plan.check_status()
            outs.append(dC.cpu().numpy())
            plan.destroy()
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
        assert g.err_norm(outs[0], g.matmul_fp64(A, B)) <= TOL_1X


def test_tma_store_is_refused_where_it_cannot_work():
    # 3xTF32 on the 256 x 64 pair tile fills shared memory with its ring and has no other form
    plan = _lib.GemmPlan(_lib.find_tile(256, 64, 2), 512, 512, 512, mode=3)
    with pytest.raises(_lib.RollerError) as e:
        plan.set_option(_lib.OPT_TMA_STORE, 1)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    plan.destroy()
    # rows of C that are not a multiple of 16 bytes long
    plan = _lib.GemmPlan(_lib.find_tile(256, 256, 2), 512, 510, 512, ldc=510, mode=3)
    with pytest.raises(_lib.RollerError) as e:
        plan.set_option(_lib.OPT_TMA_STORE, 1)
    assert e.value.status == _lib.ERR_INVALID
    plan.destroy()
    plan = _lib.GemmPlan(_lib.find_tile(256, 256, 2), 512, 512, 512, mode=3,
                         flags=_lib.FLAG_ACCUMULATE)
    with pytest.raises(_lib.RollerError) as e:
        plan.set_option(_lib.OPT_TMA_STORE, 1)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    with pytest.raises(_lib.RollerError):
        plan.set_option(99, 1)
    plan.destroy()


@pytest.mark.parametrize("tile,mode", [((256, 256, 2), 3), ((256, 128, 2), 3), ((128, 128, 1), 3),
                                       ((256, 256, 2), 1), ((128, 128, 1), 1)])
@pytest.mark.parametrize("rounds", [1, 4, -1])
def test_progressive_schedule_matches_the_oracle(tile, mode, rounds):
    """Every tile cut along K and worked through in rounds: same result within the mode's
    tolerance, on three launches in a row (the scratch slots and their flags are reused from
    round to round and from launch to launch), with and without the TMA-store output path."""
    M, N, K = 1024, 2048, 1536
    A, B = g.make_inputs(M, N, K, "uniform", seed=11)
    C64 = g.matmul_fp64(A, B)
    tol = TIGHT_3X if mode == 3 else TOL_1X
    # without the TMA-store path, with it and the tile completed by one worker, and with it
    # and the tile completed by all its workers together (the default)
    for staged, coop in (((0, 0), (1, 0), (1, 1)) if mode == 3 else ((0, 0),)):
        info = {}
        outs = run_plan(A, B, tile, mode, [(_lib.OPT_PROGRESSIVE_ROUNDS, rounds),
                                           (_lib.OPT_TMA_STORE, staged),
                                           (_lib.OPT_COOPERATIVE_FIXUP, coop)], launches=3, info=info)
        tiles = info["tiles_m"] * info["tiles_n"]
        assert info["sk_tiles"] == tiles and 1 <= info["rounds"] <= min(tiles, _lib.MAX_ROUNDS)
        if rounds > 0:
            assert info["rounds"] == rounds
        for out in outs:
            assert not np.isnan(out).any()
            assert g.err_norm(out, C64) <= tol, (tile, mode, rounds, staged, coop)
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])


def test_progressive_schedule_on_a_ragged_problem():
    M, N, K = 1111, 777, 1555
    A, B = g.make_inputs(M, N, K, "normal", seed=4)
    C64 = g.matmul_fp64(A, B)
    for tile in [(256, 128, 2), (128, 64, 1)]:
        info = {}
        out = run_plan(A, B, tile, 3, [(_lib.OPT_PROGRESSIVE_ROUNDS, 5)], launches=2, info=info)
        assert info["rounds"] == 5          # (the tile count need not be a multiple of it)
        assert g.err_norm(out[1], C64) <= TIGHT_3X


@pytest.mark.parametrize("tile", [(256, 256, 2), (128, 128, 1)])
@pytest.mark.parametrize("rounds,ratio", [(4, 60), (4, 150), (7, 40), (16, 100), (3, 400)])
def test_rounds_of_unequal_size(tile, rounds, ratio):
    """ROLLER_OPT_ROUND_RATIO: the rounds' shares of the tiles form a geometric sequence. The
    library's boundaries are the host model's (tests/test_schedule_model.py), rounds of both
    kinds (tiles completed by one worker or by all) follow each other in one launch, and the
    result is the oracle's on three launches in a row."""
    from test_schedule_model import round_tiles
    M, N, K = 1280, 2304, 1024
    A, B = g.make_inputs(M, N, K, "uniform", seed=12)
    C64 = g.matmul_fp64(A, B)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.empty(M, N, device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, mode=3)
    plan.set_option(_lib.OPT_TMA_STORE, 1)
    plan.set_option(_lib.OPT_PROGRESSIVE_ROUNDS, rounds)
    plan.set_option(_lib.OPT_ROUND_RATIO, ratio)
    tiles = -(-M // tile[0]) * -(-N // tile[1])
    assert plan.schedule_info()["rounds"] == rounds
    assert plan.round_tiles() == round_tiles(tiles, rounds, ratio)
    outs = []
    for _ in range(3):
        dC.fill_(float("nan"))
        plan.run(dA, dB, dC)
        torch.cuda.synchronize()
        plan.check_status()
        outs.append(dC.cpu().numpy())
        assert g.err_norm(outs[-1], C64) <= TIGHT_3X
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
    with pytest.raises(_lib.RollerError):
        plan.set_option(_lib.OPT_ROUND_RATIO, 10)
    plan.destroy()


def test_back_to_back_launches_with_and_without_overlap():
    """Launches that may start while the previous kernel winds down (the default) give the
    same bits as launches in plain stream order, also when consecutive kernels use the same
    stream-K scratch area and when the second GEMM reads what the first one wrote."""
    M = N = K = 1024
    A, B = g.make_inputs(M, N, K, "uniform", seed=2)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    results = []
    for overlap in (1, 0):
        p1 = _lib.GemmPlan(_lib.find_tile(128, 128, 1), M, N, K, mode=3)
        p2 = _lib.GemmPlan(_lib.find_tile(128, 64, 1), M, N, K, mode=3)
        for p in (p1, p2):
            p.set_option(_lib.OPT_OVERLAP_LAUNCH, overlap)
            p.set_stream_k(1)
        dC1 = torch.empty(M, N, device="cuda")
        dC2 = torch.empty(M, N, device="cuda")
        for _ in range(5):
            p1.run(dA, dB, dC1)      # C1 = A B
            p2.run(dC1, dB, dC2)     # C2 = C1 B: reads the previous kernel's output
            p1.run(dC2, dB, dC1)     # overwrites what the previous kernel read
            p1.run(dA, dB, dC1)
        torch.cuda.synchronize()
        p1.check_status()
        p2.check_status()
        results.append((dC1.cpu().numpy(), dC2.cpu().numpy()))
        p1.destroy()
        p2.destroy()
    assert np.array_equal(results[0][0], results[1][0])
    assert np.array_equal(results[0][1], results[1][1])
    C64 = g.matmul_fp64(A, B)
    assert g.err_norm(results[0][0], C64) <= TIGHT_3X
    assert g.err_norm(results[0][1], g.matmul_fp64(C64.astype(np.float32), B)) <= TOL_3X


def test_a_bounded_wait_that_runs_out_ends_the_kernel_with_an_error_code():
    """Stands in for the sweep's per-hint try/except (src/benchmark.py:43-58). With the test
    aid on, workers write their partial tiles but never raise the flag, so the worker that
    completes such a tile waits in vain; with a limit of 2e6 cycles (about a millisecond) the
    wait runs out, the kernel winds down and returns, the status word names the wait, and the
    host reports ROLLER_ERR_TIMEOUT. Reading the status clears it: the same plan then runs
    correctly, and so does a fresh one."""
    M, N, K = 1024, 1280, 2048          # 40 tiles of 128 x 256 on 148 workers: all cut along K
    A, B = g.make_inputs(M, N, K, "uniform", seed=8)
    C64 = g.matmul_fp64(A, B)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, N), float("nan"), device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(128, 256, 1), M, N, K, mode=3)
    plan.set_stream_k(1)
    assert plan.schedule_info()["sk_tiles"] > 0
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
    plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 1)
    plan.run(dA, dB, dC)
    torch.cuda.synchronize()            # returns: the kernel ended by itself
    assert plan.device_status() == _lib.DEV_TIMEOUT_FIXUP
    assert plan.device_status() == 0    # read and cleared
    # the same plan, test aid off, default limit: correct again
    plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 0)
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0)
    dC.fill_(float("nan"))
    plan.run(dA, dB, dC)
    torch.cuda.synchronize()
    plan.check_status()
    assert g.err_norm(dC.cpu().numpy(), C64) <= TIGHT_3X
    # check_status raises for a failed launch, which is what the sweep's try/except catches
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
    plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 1)
    plan.run(dA, dB, dC)
    with pytest.raises(_lib.RollerError) as e:
        plan.check_status()
    assert e.value.status == _lib.ERR_TIMEOUT
    plan.destroy()
    fresh = _lib.GemmPlan(_lib.find_tile(256, 256, 2), M, N, K, mode=3)
    dC.fill_(float("nan"))
    fresh.run(dA, dB, dC)
    torch.cuda.synchronize()
    fresh.check_status()
    assert g.err_norm(dC.cpu().numpy(), C64) <= TIGHT_3X
    fresh.destroy()


def test_a_wait_runs_out_in_the_cooperative_completion_of_a_tile():
    """The progressive schedule with tiles completed by all their workers: with the flags
    withheld every worker waits in vain for the others' partial sums, gives up after the limit,
    and the launch ends with the same error code; afterwards the plan works."""
    M, N, K = 1024, 2048, 2048
    A, B = g.make_inputs(M, N, K, "uniform", seed=10)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.empty(M, N, device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(256, 256, 2), M, N, K, mode=3)
    plan.set_option(_lib.OPT_TMA_STORE, 1)
    plan.set_option(_lib.OPT_PROGRESSIVE_ROUNDS, 4)
    assert plan.schedule_info()["rounds"] == 4
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
    plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 1)
    plan.run(dA, dB, dC)
    torch.cuda.synchronize()
    # (whichever role's wait ran out first has recorded its code: the workers waiting for the
    # partial sums, or the producer and MMA issuer stalled behind them)
    assert plan.device_status() != 0
    plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 0)
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0)
    for _ in range(2):
        dC.fill_(float("nan"))
        plan.run(dA, dB, dC)
        torch.cuda.synchronize()
        plan.check_status()
        assert g.err_norm(dC.cpu().numpy(), g.matmul_fp64(A, B)) <= TIGHT_3X
    plan.destroy()


def test_a_cta_pair_winds_down_together_when_a_wait_runs_out():
    """The same failure on a kernel whose CTAs work in pairs: both CTAs of a pair meet at a
    cluster barrier before they release tensor memory, so both must reach it."""
    M, N, K = 1024, 2304, 2048          # 36 pair tiles on 74 pairs: all cut along K
    A, B = g.make_inputs(M, N, K, "uniform", seed=9)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.empty(M, N, device="cuda")
    for mode in (3, 1):
        plan = _lib.GemmPlan(_lib.find_tile(256, 256, 2), M, N, K, mode=mode)
        plan.set_stream_k(1)
        assert plan.schedule_info()["sk_tiles"] > 0
        plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
        plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 1)
        plan.run(dA, dB, dC)
        torch.cuda.synchronize()
        assert plan.device_status() == _lib.DEV_TIMEOUT_FIXUP
        plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 0)
        plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0)
        plan.run(dA, dB, dC)
        torch.cuda.synchronize()
        plan.check_status()
        err = g.err_norm(dC.cpu().numpy(), g.matmul_fp64(A, B))
        assert err <= (TIGHT_3X if mode == 3 else TOL_1X)
        plan.destroy()


def test_best_hint_skips_a_kernel_that_gave_up(monkeypatch):
    """The measured-feedback search must not crown a kernel that ended early: timing raises for
    a launch whose wait ran out, and the hint is skipped like one that failed to compile."""
    from mlir_roller_b200 import roller
    from mlir_roller_b200.analyze import MatmulConfig
    cfg = MatmulConfig(1024, 1280, 2048, 32)
    real_compile = roller.Compiler.compile
    sabotaged = []

    def compile_and_sabotage_first(self):
        fn = real_compile(self)
        if not sabotaged:
            sabotaged.append(tuple(self.hint.block_tile))
            fn.plan.set_stream_k(1)
            if fn.plan.schedule_info()["sk_tiles"] > 0:
                fn.plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
                fn.plan.set_option(_lib.OPT_TEST_DROP_PUBLISH, 1)
            else:
                sabotaged.append("not split")
        return fn

    monkeypatch.setattr(roller.Compiler, "compile", compile_and_sabotage_first)
    hint, fn, ms = roller.best_hint(cfg, topk=4, mode=3)
    assert ms > 0
    if "not split" not in sabotaged:
        assert tuple(hint.block_tile) != sabotaged[0]
    fn.plan.destroy()


def test_arrival_flags_signal_and_bounded_wait():
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    base = flags.data_ptr()
    _lib.flag_signal_async([base + 4 * 1, base + 4 * 5], 7)
    _lib.flag_wait_async(base, 64, (1 << 1) | (1 << 5), 7, status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and flags[1].item() == 7 and flags[5].item() == 7
    assert int(flags.sum().item()) == 14
    # a later value satisfies an earlier wait (flags count steps)
    _lib.flag_wait_async(base, 64, 1 << 5, 3, status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # word 9 is never raised: the wait gives up after ~2e6 cycles and says so
    _lib.flag_wait_async(base, 64, (1 << 1) | (1 << 9), 7, status.data_ptr(), limit_cycles=2_000_000)
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.DEV_TIMEOUT_PEER
    with pytest.raises(_lib.RollerError):
        _lib.flag_signal_async([base + 2], 1)           # misaligned word
    with pytest.raises(_lib.RollerError):
        _lib.flag_signal_async([base] * 40, 1)          # more targets than one call takes


@pytest.mark.parametrize("tile,rounds", [((256, 256, 2), 0), ((256, 256, 2), 4), ((128, 128, 1), 2)])
def test_a_launch_that_does_its_own_hand_shake(tile, rounds):
    """roller_b200_gemm_run_synced on one GPU, both flags in local memory: with "go" already
    raised the result is the plain launch's and the arrival word holds the step afterwards; a
    later "go" value also satisfies the wait; with "go" never raised the wait in front of the
    first store runs out after about a millisecond, the launch is reported as failed and
    raises no arrival flag; the plan is usable afterwards."""
    M, N, K = 1024, 1536, 1024
    A, B = g.make_inputs(M, N, K, "uniform", seed=21)
    C64 = g.matmul_fp64(A, B)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, N), float("nan"), device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    go, arrive = flags.data_ptr(), flags.data_ptr() + 16
    plan = _lib.GemmPlan(_lib.find_tile(*tile), M, N, K, mode=3)
    plan.set_option(_lib.OPT_TMA_STORE, 1)
    if rounds:
        plan.set_option(_lib.OPT_PROGRESSIVE_ROUNDS, rounds)
    ptrs = (dA.data_ptr(), dB.data_ptr(), dC.data_ptr())
    for step, go_now in ((1, 0), (2, 1), (3, 5)):
        flags[0] = go_now
        dC.fill_(float("nan"))
        torch.cuda.synchronize()
        plan.run_synced_ptr(*ptrs, go_ptr=go if step > 1 else 0, go_value=step - 1,
                            arrive_ptr=arrive, arrive_value=step)
        torch.cuda.synchronize()
        plan.check_status()
        assert int(flags[4].item()) == step
        assert g.err_norm(dC.cpu().numpy(), C64) <= TIGHT_3X
    # without an arrival flag: only the wait for "go"
    plan.run_synced_ptr(*ptrs, go_ptr=go, go_value=5)
    torch.cuda.synchronize()
    plan.check_status()
    assert int(flags[4].item()) == 3
    # "go" = 9 never comes
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 2_000_000)
    plan.run_synced_ptr(*ptrs, go_ptr=go, go_value=9, arrive_ptr=arrive, arrive_value=4)
    torch.cuda.synchronize()
    st = plan.device_status()
    # (with tiles shared between workers, one waiting for another's partial sums may be the
    # first whose limit runs out: the code then names that wait)
    assert st == _lib.DEV_TIMEOUT_PEER or (rounds and st != 0)
    assert int(flags[4].item()) == 3                # no arrival from a failed launch
    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0)
    flags[0] = 9
    dC.fill_(float("nan"))
    torch.cuda.synchronize()
    plan.run_synced_ptr(*ptrs, go_ptr=go, go_value=9, arrive_ptr=arrive, arrive_value=4)
    torch.cuda.synchronize()
    plan.check_status()
    assert int(flags[4].item()) == 4
    assert g.err_norm(dC.cpu().numpy(), C64) <= TIGHT_3X
    plan.destroy()


def test_the_hand_shake_needs_the_tma_store_path():
    M, N, K = 256, 250, 128        # rows of C are not multiples of 16 bytes: no TMA stores
    dA = torch.zeros(M, K, device="cuda")
    dB = torch.zeros(K, N, device="cuda")
    dC = torch.zeros(M, N, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(128, 128, 1), M, N, K, mode=3)
    with pytest.raises(_lib.RollerError) as e:
        plan.run_synced_ptr(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                            arrive_ptr=flags.data_ptr(), arrive_value=1)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    with pytest.raises(_lib.RollerError) as e:
        plan.run_synced_ptr(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                            arrive_ptr=flags.data_ptr() + 2, arrive_value=1)
    assert e.value.status == _lib.ERR_INVALID
    plan.destroy()


def test_early_exit_leaves_the_result_alone():
    """ROLLER_OPT_EARLY_EXIT: CTAs leave once the TMA unit has read their last tile from shared
    memory; C is complete when the kernel is. Same bits as without the option, launch after
    launch, also with rounds; a launch that raises an arrival flag still waits for its stores."""
    M, N, K = 1024, 1536, 1024
    A, B = g.make_inputs(M, N, K, "uniform", seed=23)
    ref = run_plan(A, B, (256, 256, 2), 3, [(_lib.OPT_TMA_STORE, 1)])[0]
    for opts in ([], [(_lib.OPT_PROGRESSIVE_ROUNDS, 2), (_lib.OPT_ROUND_RATIO, 40)]):
        plain = run_plan(A, B, (256, 256, 2), 3, [(_lib.OPT_TMA_STORE, 1)] + opts, launches=2)
        early = run_plan(A, B, (256, 256, 2), 3, [(_lib.OPT_TMA_STORE, 1), (_lib.OPT_EARLY_EXIT, 1)] + opts,
                         launches=3)
        for out in early:
            assert np.array_equal(out, plain[0])
        assert g.err_norm(plain[0], g.matmul_fp64(A, B)) <= TIGHT_3X
    assert g.err_norm(ref, g.matmul_fp64(A, B)) <= TIGHT_3X
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, N), float("nan"), device="cuda")
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    plan = _lib.GemmPlan(_lib.find_tile(256, 256, 2), M, N, K, mode=3)
    plan.set_option(_lib.OPT_TMA_STORE, 1)
    plan.set_option(_lib.OPT_EARLY_EXIT, 1)
    plan.run_synced_ptr(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), arrive_ptr=flags.data_ptr(),
                        arrive_value=7)
    torch.cuda.synchronize()
    plan.check_status()
    assert int(flags[0].item()) == 7 and np.array_equal(dC.cpu().numpy(), ref)
    plan.destroy()
