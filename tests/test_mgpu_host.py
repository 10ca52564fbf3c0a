"""Host-side logic of the multi-GPU driver: partitioning and the gather, the latter over a
world_size-2 gloo group on CPU (blocks produced by the oracle stand in for the kernel output)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from hypothesis import given, settings, strategies as st

from mlir_roller_b200 import mgpu


def test_row_partition_of_m13():
    blocks = mgpu.partition(8192, 4096, 8, 1)
    assert [(b.row0, b.row1, b.col0, b.col1) for b in blocks] == \
        [(i * 1024, (i + 1) * 1024, 0, 4096) for i in range(8)]
    assert [b.rank for b in blocks] == list(range(8))


def test_2d_partition_of_16384():
    blocks = mgpu.partition(16384, 16384, 4, 2)
    assert len(blocks) == 8
    b = blocks[5]  # i = 2, j = 1
    assert (b.row0, b.row1, b.col0, b.col1) == (8192, 12288, 8192, 16384)
    assert all(b.rows == 4096 and b.cols == 8192 for b in blocks)


def test_default_grid():
    assert mgpu.default_grid(8, 8192, 4096) == (8, 1)
    assert mgpu.default_grid(8, 16384, 16384) == (8, 1)
    assert mgpu.default_grid(8, 2048, 2048) == (4, 2)
    assert mgpu.default_grid(1, 100, 100) == (1, 1)


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 5000), st.integers(1, 5000), st.integers(1, 8), st.integers(1, 4))
def test_partition_tiles_c_exactly(M, N, gm, gn):
    blocks = mgpu.partition(M, N, gm, gn)
    assert len(blocks) == gm * gn
    cover = np.zeros((M, N), dtype=np.int8)
    for b in blocks:
        assert 0 <= b.row0 <= b.row1 <= M and 0 <= b.col0 <= b.col1 <= N
        if b.rows and b.cols:
            assert b.row0 % 128 == 0 and b.col0 % 32 == 0
        cover[b.row0:b.row1, b.col0:b.col1] += 1
    assert (cover == 1).all()


def test_partition_rejects_bad_grid():
    with pytest.raises(ValueError):
        mgpu.partition(10, 10, 0, 1)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather_worker(rank, world, port, grid, M, N, K, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import gemm_oracle
        A, B = gemm_oracle.make_inputs(M, N, K, "uniform", seed=3)
        blocks = mgpu.partition(M, N, grid[0], grid[1], align_m=8, align_n=4)
        b = blocks[rank]
        local = torch.from_numpy(gemm_oracle.matmul_fp32(A[b.row0:b.row1], B[:, b.col0:b.col1]))
        sentinel = torch.full((M, N), float("nan"))
        full = mgpu.gather_blocks(local, blocks, M, N, rank, root=0, out=sentinel)
        if rank == 0:
            want = np.empty((M, N), np.float32)
            for bb in blocks:
                want[bb.row0:bb.row1, bb.col0:bb.col1] = gemm_oracle.matmul_fp32(
                    A[bb.row0:bb.row1], B[:, bb.col0:bb.col1])
            q.put(bool(np.array_equal(full.numpy(), want)) and full is sentinel)
        else:
            q.put(full is None)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("grid", [(2, 1), (1, 2)])
def test_gather_two_ranks_gloo(grid):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, grid, 40, 24, 16, q))
             for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(results)


def test_gather_checks_block_shape():
    blocks = mgpu.partition(16, 16, 1, 1, align_m=8, align_n=4)
    with pytest.raises(ValueError):
        mgpu.gather_blocks(torch.zeros(3, 3), blocks, 16, 16, rank=0)


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 4096), st.integers(0, 9000), st.integers(1, 9), st.booleans())
def test_bands_tile_the_block(row0, rows, bands, taper):
    out = mgpu.split_bands(row0, row0 + rows, bands, taper=taper)
    assert len(out) <= bands
    if rows == 0:
        assert out == []
        return
    assert out[0][0] == row0 and out[-1][1] == row0 + rows
    for (a0, a1), (b0, b1) in zip(out, out[1:]):
        assert a1 == b0
    for r0, r1 in out:
        assert r1 > r0 and (r0 - row0) % 256 == 0
    if taper:       # later bands are never larger (in tile rows) than earlier ones
        units = [-(-(r1 - r0) // 256) for r0, r1 in out]
        assert units == sorted(units, reverse=True)
        if rows >= 256 * bands:
            assert len(out) == bands


def test_bands_of_a_16384_row_shard():
    assert mgpu.split_bands(2048, 4096, 4) == [(2048, 2560), (2560, 3072), (3072, 3584), (3584, 4096)]
    assert mgpu.split_bands(0, 1000, 4) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert mgpu.split_bands(0, 4096, 4, taper=True) == [(0, 1792), (1792, 3072), (3072, 3840), (3840, 4096)]
    assert mgpu.split_bands(0, 2048, 4, taper=True) == [(0, 768), (768, 1536), (1536, 1792), (1792, 2048)]
    with pytest.raises(ValueError):
        mgpu.split_bands(0, 10, 0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_push_order(world):
    orders = [mgpu.push_order(r, world, "all") for r in range(world)]
    for r, o in enumerate(orders):
        assert sorted(o) == [x for x in range(world) if x != r]
    # at every step of the rotation the ranks write to pairwise different destinations
    for step in range(world - 1):
        assert len({o[step] for o in orders}) == world
    assert mgpu.push_order(0, world, "root") == []
    if world > 1:
        assert mgpu.push_order(1, world, "root") == [0]
        assert mgpu.push_order(0, world, "root", root=1) == [1]
    with pytest.raises(ValueError):
        mgpu.push_order(0, world, "ring")


def test_default_bands():
    assert mgpu.default_bands(2048, 16384) == 4
    assert mgpu.default_bands(4096, 4096) == 2
    assert mgpu.default_bands(1024, 4096) == 2
    assert mgpu.default_bands(512, 1024) == 1


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 1500), st.integers(1, 700), st.integers(1, 300), st.sampled_from([1, 2, 4, 8]),
       st.integers(1, 5), st.sampled_from(["root", "all"]), st.booleans())
def test_band_schedule_delivers_every_block(M, N, K, world, bands, dest, two_d):
    """Replay every rank's schedule on flat host arrays (the 'kernel' writes the band into the
    rank's own C, each push copies it to the destination's C at the same offset): afterwards
    rank 0 -- or every rank -- holds the whole matrix, and no step reads outside its operands."""
    grid = (world // 2, 2) if (two_d and world % 2 == 0) else (world, 1)
    blocks = mgpu.partition(M, N, grid[0], grid[1], align_m=256)
    truth = np.arange(M * N, dtype=np.float64).reshape(M, N)
    Cs = [np.full(M * N, -1.0) for _ in range(world)]
    for r, b in enumerate(blocks):
        steps = mgpu.band_schedule(b, N, K, bands, mgpu.push_order(r, world, dest))
        assert len(steps) <= bands
        assert sum(s.row1 - s.row0 for s in steps) == (b.rows if b.cols else 0)
        for s in steps:
            rows = s.row1 - s.row0
            assert 0 <= s.a_off and s.a_off + rows * K <= max(b.rows, 1) * K   # inside A[rows of block]
            assert s.b_off == b.col0 and s.b_off + s.cols <= N
            assert s.c_off == s.row0 * N + b.col0
            for i in range(rows):       # the band, row by row, with leading dimension N
                lo = s.c_off + i * N
                Cs[r][lo:lo + s.cols] = truth[s.row0 + i, b.col0:b.col0 + s.cols]
                for d in s.dests:
                    assert d != r
                    Cs[d][lo:lo + s.cols] = Cs[r][lo:lo + s.cols]
    holders = range(world) if dest == "all" else [0]
    for r in holders:
        assert np.array_equal(Cs[r].reshape(M, N), truth)


def test_run_near_gpu_changes_nothing_when_the_topology_cannot_be_read(monkeypatch):
    """Without a GPU (or without the sysfs entries) the helper reports None and leaves the
    process's CPU affinity alone; with a readable topology it narrows the affinity to the
    GPU's NUMA node."""
    import builtins
    import io
    import os
    import types

    import torch

    before = os.sched_getaffinity(0)
    assert mgpu.run_near_gpu(0) is None or not torch.cuda.is_available()
    assert os.sched_getaffinity(0) == before
    # a fake machine: GPU 0 at 0000:1b:00.0 on node 1, whose cores are the ones we may use
    cpus = sorted(before)
    keep = cpus[: max(1, len(cpus) // 2)]
    files = {"/sys/bus/pci/devices/0000:1b:00.0/numa_node": "1\n",
             "/sys/devices/system/node/node1/cpulist": ",".join(str(c) for c in keep) + "\n"}
    real_open = builtins.open

    def fake_open(path, *a, **k):
        if path in files:
            return io.StringIO(files[path])
        return real_open(path, *a, **k)

    monkeypatch.setattr(builtins, "open", fake_open)
    monkeypatch.setattr(torch.cuda, "get_device_properties",
                        lambda i: types.SimpleNamespace(pci_bus_id="00000000:1B:00.0"))
    try:
        assert mgpu.run_near_gpu(0) == 1
        assert os.sched_getaffinity(0) == set(keep)
        os.sched_setaffinity(0, before)
        # the same device described by numbers, as torch reports it
        monkeypatch.setattr(torch.cuda, "get_device_properties",
                            lambda i: types.SimpleNamespace(pci_bus_id=0x1B, pci_device_id=0,
                                                            pci_domain_id=0))
        assert mgpu.run_near_gpu(0) == 1
        assert os.sched_getaffinity(0) == set(keep)
    finally:
        os.sched_setaffinity(0, before)


def test_round_shape_of_the_fused_exchange():
    """The rounds of a kernel whose C leaves over NVLink while it computes, by the size of the
    block: none for many waves; for one to four waves two shrinking
    rounds when the computation is the longer of the two and four growing ones when the link
    is; four equal rounds below one wave; explicit values win."""
    from mlir_roller_b200 import mgpu
    gb = 690e6        # bytes the link moves per millisecond at the measured rate
    assert mgpu.fused_round_shape(int(0.6 * gb), 1.0, 128, 74) == (2, 40)
    assert mgpu.fused_round_shape(int(1.2 * gb), 1.0, 128, 74) == (4, 160)
    assert mgpu.fused_round_shape(int(1.2 * gb), 1.0, 64, 74) == (4, 100)     # less than one wave
    assert mgpu.fused_round_shape(int(0.3 * gb), 1.0, 64, 74) == (4, 100)
    assert mgpu.fused_round_shape(int(0.4 * gb), 1.0, 512, 74) == (0, 100)    # whole tiles, wave after wave
    assert mgpu.fused_round_shape(int(1.2 * gb), 1.0, 128, 74, rounds=8, round_ratio=100) == (8, 100)
    assert mgpu.fused_round_shape(int(0.6 * gb), 1.0, 128, 74, rounds=3) == (3, 40)
    assert mgpu.fused_round_shape(int(gb), 0.0, 128, 74) == (4, 160)  # no time estimate: link-bound
    assert mgpu.fused_round_shape(0, 1.0, 128, 74) == (2, 40)
