"""Worker for test_overlap_gpu.py: one process per GPU (launched through torch.distributed.run),
checks mgpu.OverlappedGemm -- bands pushed into the destination ranks' C over symmetric memory,
or tiles stored there by the kernel itself -- and mgpu.HostStagedGemm against an fp64 product.
Exits non-zero on any mismatch."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mlir_roller_b200 import mgpu  # noqa: E402

TOL_3X = 1e-5


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    M, N, K = 2048, 1024, 640
    g = torch.Generator(device="cuda")
    g.manual_seed(5)                       # the same A and B on every rank
    A = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
    B = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
    ref = A.double() @ B.double()
    scale = float(ref.abs().max())
    grids = [(world, 1)] + ([(1, world), (2, world // 2)] if world % 2 == 0 else [])
    bad = 0
    for grid in grids:
        for dest, bands, fused in (("root", 1, False), ("root", 3, False), ("all", 1, False),
                                   ("all", 3, False), ("root", 3, True)):
            og = mgpu.OverlappedGemm(M, N, K, rank, world, grid=grid, bands=bands, dest=dest,
                                     taper=(bands == 3), fused=fused)
            assert og.handle.multicast_ptr == 0
            b = og.block
            og.C.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(2):          # twice: the second step overwrites the first
                og.run(A[b.row0:b.row1].contiguous(), B)
                og.finish()
                torch.cuda.synchronize()
                dist.barrier()
            for p in og.plans:
                p.check_status()
            if dest == "all" or rank == 0:
                err = float((og.C.double() - ref).abs().max()) / scale
            elif fused:                 # nothing is written locally: the block went to rank 0
                err = 0.0
            else:                       # only this rank's own block is defined
                err = float((og.C[b.row0:b.row1, b.col0:b.col1].double()
                             - ref[b.row0:b.row1, b.col0:b.col1]).abs().max()) / scale \
                    if b.rows * b.cols else 0.0
            ok = err <= TOL_3X          # NaN compares false
            if not ok:
                bad += 1
            print(f"rank {rank} grid {grid} dest {dest} bands {bands} fused {fused}: err {err:.2e} "
                  f"{'ok' if ok else 'FAIL'}", flush=True)
            og.destroy()
            del og
            dist.barrier()
    # two C buffers in flight: the senders work on step s + 1 while rank 0 still reads step s.
    # Five steps with different operands and no host synchronisation between them; rank 0 copies
    # every step's C on the stream between the arrival wait and the release of the buffer.
    og = mgpu.OverlappedGemm(M, N, K, rank, world, grid=(world, 1), dest="root", fused=True, depth=2)
    b = og.block
    As = [(A[b.row0:b.row1] * (s + 1)).contiguous() for s in range(5)]
    got = []
    for s in range(5):
        og.run(As[s], B)
        og.finish(release=False)
        if rank == 0:
            got.append(og.C.clone())
        og.release()
    torch.cuda.synchronize()
    dist.barrier()
    og.check_status()
    err = max((float((c.double() - (s + 1) * ref).abs().max()) / ((s + 1) * scale)
               for s, c in enumerate(got)), default=0.0)
    ok = err <= TOL_3X and len({c.data_ptr() for c in og.C_bufs}) == 2
    print(f"rank {rank} fused, two C buffers, 5 steps: err {err:.2e} {'ok' if ok else 'FAIL'}", flush=True)
    bad += 0 if ok else 1
    og.destroy()
    del og, got
    dist.barrier()
    # the same exchange with bf16 operands (the band offsets into A and B are in elements)
    A16, B16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
    ref16 = A16.double() @ B16.double()
    og = mgpu.OverlappedGemm(M, N, K, rank, world, grid=(world, 1), bands=3, dest="all", mode=16)
    b = og.block
    og.run(A16[b.row0:b.row1].contiguous(), B16)
    og.finish()
    torch.cuda.synchronize()
    dist.barrier()
    err = float((og.C.double() - ref16).abs().max()) / float(ref16.abs().max())
    print(f"rank {rank} bf16 dest all bands 3: err {err:.2e} {'ok' if err <= TOL_3X else 'FAIL'}", flush=True)
    bad += 0 if err <= TOL_3X else 1
    og.destroy()
    del og
    dist.barrier()
    # operands in host memory: each rank uploads its rows of A and a 1/world share of B's rows,
    # the shares are exchanged over NVLink, C comes back to the host
    rows = M // world
    hs = mgpu.HostStagedGemm(rows, N, K, rank, world)
    hA = A[rank * rows:(rank + 1) * rows].cpu().pin_memory()
    hB = B.cpu().pin_memory()
    hC = torch.full((rows, N), float("nan")).pin_memory()
    for _ in range(2):
        hs.run(hA, hB, hC)
        torch.cuda.synchronize()
    hs.plan.check_status()
    err = float((hC.double() - ref[rank * rows:(rank + 1) * rows].cpu()).abs().max()) / scale
    up, down = hs.bytes_per_call()
    ok = err <= TOL_3X and up == 4 * (rows * K + (K // world) * N) and down == 4 * rows * N
    print(f"rank {rank} host-staged: err {err:.2e} h2d {up} d2h {down} {'ok' if ok else 'FAIL'}", flush=True)
    bad += 0 if ok else 1
    hs.destroy()
    dist.barrier()
    t = torch.tensor([bad], device="cuda")
    dist.all_reduce(t)
    dist.destroy_process_group()
    return 1 if int(t.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
