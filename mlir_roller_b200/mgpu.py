"""Output-stationary sharding of one GEMM across the GPUs of a node.

The reference is single-GPU (it pins one device, .env:5-6); this driver is what the B200 build
adds on top of its hot path. One process per GPU (`torch.distributed`, NCCL over NVLink): rank r
owns one block of C and computes it from its rows of A and its columns of B with the full
reduction, so the compute phase needs no exchange at all. Operands are replicated (or placed)
in every GPU's own memory before the timed region. A collective is used only to bring the C
blocks to one rank when the caller wants the whole matrix there.

Layouts
  * 1-D row sharding (grid = (n, 1)): rank r holds A[rows_r, :], all of B, and C[rows_r, :].
  * 2-D sharding (grid = (gm, gn)): rank r = i * gn + j holds A[rows_i, :], reads the column
    block B[:, cols_j] as a strided view of the replicated B (ldb stays N; TMA handles the
    stride, nothing is repacked), and owns C[rows_i, cols_j].
The rTile search runs per shard shape, so every rank picks the kernel that suits its block.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class Block:
    """Half-open row/column ranges of C owned by one rank."""
    rank: int
    row0: int
    row1: int
    col0: int
    col1: int

    @property
    def rows(self) -> int:
        return self.row1 - self.row0

    @property
    def cols(self) -> int:
        return self.col1 - self.col0


def _el_bits(mode: int) -> int:
    """Operand width of an arithmetic mode: 16 for the bf16 / fp16 modes, else 32."""
    return 16 if mode in (16, 17) else 32


def _split(extent: int, parts: int, align: int) -> List[Tuple[int, int]]:
    """Cut [0, extent) into `parts` contiguous ranges whose boundaries are multiples of
    `align` (except the end); earlier ranges take the remainder units. Ranges may be empty
    when there are fewer units than parts."""
    units = -(-extent // align)
    base, extra = divmod(units, parts)
    out, start = [], 0
    for p in range(parts):
        n = (base + (1 if p < extra else 0)) * align
        stop = min(start + n, extent)
        out.append((start, stop))
        start = stop
    return out


def partition(M: int, N: int, grid_m: int, grid_n: int, align_m: int = 128,
              align_n: int = 32) -> List[Block]:
    """Blocks of C for a grid_m x grid_n process grid, rank = i * grid_n + j.

    Row boundaries fall on multiples of `align_m` (one CTA's tile rows) and column boundaries
    on multiples of `align_n` (one TMA box of B, which also keeps the B view 16-byte aligned).
    """
    if grid_m < 1 or grid_n < 1:
        raise ValueError("grid dimensions must be positive")
    rows = _split(M, grid_m, align_m)
    cols = _split(N, grid_n, align_n)
    return [Block(i * grid_n + j, r0, r1, c0, c1)
            for i, (r0, r1) in enumerate(rows) for j, (c0, c1) in enumerate(cols)]


def default_grid(world_size: int, M: int, N: int) -> Tuple[int, int]:
    """Row sharding while blocks stay at least 1024 rows tall, else the most square grid
    (8 ranks on a square problem -> 4 x 2)."""
    if M // world_size >= 1024 or world_size == 1:
        return world_size, 1
    best = (world_size, 1)
    for gn in range(1, world_size + 1):
        if world_size % gn == 0:
            gm = world_size // gn
            if abs(M / gm - N / gn) < abs(M / best[0] - N / best[1]):
                best = (gm, gn)
    return best


def gather_blocks(local, blocks: Sequence[Block], M: int, N: int, rank: int, root: int = 0,
                  group=None, out=None):
    """Assemble C on `root` from every rank's block. `local` is this rank's (rows x cols) block,
    contiguous. Returns the full matrix on root (written into `out` when given), None elsewhere.

    Uses point-to-point sends into `root` (NCCL send/recv on GPUs, gloo on CPU): blocks differ
    in shape, and only one rank needs the result, so an all-gather would move 7/8 of the data
    for nothing on an 8-GPU node.
    """
    import torch
    import torch.distributed as dist

    mine = blocks[rank]
    if tuple(local.shape) != (mine.rows, mine.cols):
        raise ValueError(f"rank {rank}: block is {tuple(local.shape)}, expected {(mine.rows, mine.cols)}")
    if rank != root:
        if mine.rows * mine.cols > 0:
            for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, local.contiguous(), root,
                                                          group=group)]):
                req.wait()
        return None
    full = out if out is not None else torch.empty((M, N), dtype=local.dtype, device=local.device)
    full[mine.row0:mine.row1, mine.col0:mine.col1].copy_(local)
    ops, staged = [], []
    for b in blocks:
        if b.rank == root or b.rows * b.cols == 0:
            continue
        if b.col0 == 0 and b.col1 == N:
            # a band of whole rows is contiguous in C: receive in place
            ops.append(dist.P2POp(dist.irecv, full[b.row0:b.row1], b.rank, group=group))
        else:
            tmp = torch.empty((b.rows, b.cols), dtype=local.dtype, device=local.device)
            ops.append(dist.P2POp(dist.irecv, tmp, b.rank, group=group))
            staged.append((b, tmp))
    if ops:
        # one batch: all senders stream into the root at once instead of one after another
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for b, tmp in staged:
        full[b.row0:b.row1, b.col0:b.col1].copy_(tmp)
    return full


class ShardedGemm:
    """This rank's part of C = A @ B on a grid_m x grid_n process grid.

    Usage, one process per GPU with the process group already initialised:

        sg = ShardedGemm(M, N, K, rank, world_size)            # searches the shard's rTile
        sg.run(A_rows, B_full, C_block)                         # local kernel, no communication
        C = sg.gather(C_block)                                  # whole C on rank 0, None elsewhere
    """

    def __init__(self, M: int, N: int, K: int, rank: int, world_size: int,
                 grid: Optional[Tuple[int, int]] = None, mode: int = 3, arch=None,
                 measure: bool = False):
        from . import _lib, roller
        from .analyze import MatmulConfig
        self.M, self.N, self.K = M, N, K
        self.rank, self.world_size = rank, world_size
        self.grid = grid if grid is not None else default_grid(world_size, M, N)
        if self.grid[0] * self.grid[1] != world_size:
            raise ValueError(f"grid {self.grid} does not match world size {world_size}")
        self.blocks = partition(M, N, self.grid[0], self.grid[1])
        self.block = self.blocks[rank]
        self.mode = mode
        self.plan = None
        self.hint = None
        if self.block.rows > 0 and self.block.cols > 0:
            cfg = MatmulConfig(self.block.rows, self.block.cols, K, _el_bits(mode))
            hint, _fn, _ms = roller.best_hint(cfg, arch, mode=mode, measure=measure)
            self.hint = hint
            tile = roller.kernel_tile_for(hint)
            # B is addressed inside the replicated K x N matrix, C is this rank's own block
            self.plan = _lib.GemmPlan(tile, self.block.rows, self.block.cols, K, lda=K, ldb=N,
                                      ldc=self.block.cols, mode=mode)

    def local_operands(self, A_full, B_full):
        """Views of the replicated operands this rank reads: its rows of A, its columns of B."""
        b = self.block
        return A_full[b.row0:b.row1], B_full[:, b.col0:b.col1]

    def run(self, A_rows, B_full, C_block, stream=None) -> None:
        """Enqueue the local GEMM. `A_rows` = A[rows_r, :] (contiguous), `B_full` = the whole
        replicated B (K x N, contiguous), `C_block` = this rank's rows x cols output."""
        if self.plan is None:
            return
        b = self.block
        elem = B_full.element_size()
        self.plan.run_ptr(A_rows.data_ptr(), B_full.data_ptr() + b.col0 * elem,
                          C_block.data_ptr(), stream)

    def gather(self, C_block, root: int = 0, group=None, out=None):
        return gather_blocks(C_block, self.blocks, self.M, self.N, self.rank, root, group, out)

    def flops(self) -> int:
        return 2 * self.block.rows * self.block.cols * self.K


def run_near_gpu(device_index: int) -> Optional[int]:
    """Restrict this process to the CPU cores of the NUMA node its GPU hangs off, so that host
    buffers it allocates (and pins) afterwards are placed in that node's memory by first touch
    and its copies do not cross the socket interconnect. With one process per GPU and all of
    them uploading at once that is where the host side saturates first. Returns the node, or
    None when the topology cannot be read (nothing is changed then)."""
    import os
    try:
        import torch
        props = torch.cuda.get_device_properties(device_index)
        bus = props.pci_bus_id
        if isinstance(bus, str):                  # "00000000:1B:00.0"
            bdf = bus.lower()
        else:                                     # numbers: domain, bus, device
            bdf = f"{props.pci_domain_id:04x}:{bus:02x}:{props.pci_device_id:02x}.0"
    except Exception:  # noqa: BLE001 - no GPU, or a torch without these properties
        bdf = None
    try:
        if bdf is None:
            return None
        if len(bdf.split(":")[0]) == 8:          # 00000000:1b:00.0 -> 0000:1b:00.0
            bdf = bdf[4:]
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError):
        return None


class HostStagedGemm:
    """This rank's C block = A_rows @ B with all three matrices in (pinned) host memory, on a node
    whose ranks all need the same B.

    The reference uploads both operands of every GEMM from the host (src/roller.py:532-534). With
    one process per GPU, doing the same on every rank would push `world` copies of B through the
    host's PCIe links. Here a rank uploads its own rows of A and only its 1/world share of B's
    rows; the shares are exchanged between the GPUs over NVLink (an in-place NCCL all-gather into
    the rank's B buffer), which is more than ten times faster than the host link, and the kernel
    follows on the same stream. C is read back into host memory at the end. Everything is
    enqueued on the given stream; the caller synchronises.
    """

    def __init__(self, rows: int, N: int, K: int, rank: int, world_size: int, mode: int = 3,
                 group=None, arch=None, measure: bool = False, tile=None):
        import torch
        import torch.distributed as dist
        from . import _lib, roller
        from .analyze import MatmulConfig
        if K % world_size:
            raise ValueError("B's rows are exchanged in equal shares: K must divide by the world size")
        self.rows, self.N, self.K = rows, N, K
        self.rank, self.world_size, self.mode = rank, world_size, mode
        self.group = group if group is not None else dist.group.WORLD
        self._torch, self._dist = torch, dist
        dt = roller.operand_dtype(mode)
        if tile is None:
            hint, _fn, _ms = roller.best_hint(MatmulConfig(rows, N, K, _el_bits(mode)), arch,
                                              mode=mode, measure=measure)
            tile = roller.kernel_tile_for(hint)
        self.plan = _lib.GemmPlan(tile, rows, N, K, mode=mode)
        self.dA = torch.empty(rows, K, dtype=dt, device="cuda")
        self.dB = torch.empty(K, N, dtype=dt, device="cuda")
        self.dC = torch.empty(rows, N, dtype=torch.float32, device="cuda")
        share = K // world_size
        self.share = (rank * share, (rank + 1) * share)

    def bytes_per_call(self):
        """(host-to-device, device-to-host) bytes one `run` moves over this rank's host link."""
        eb = self.dA.element_size()
        return (eb * (self.rows * self.K + (self.share[1] - self.share[0]) * self.N),
                4 * self.rows * self.N)

    def run(self, hA, hB, hC, stream=None) -> None:
        """hA: this rank's rows of A, hB: the whole B, hC: receives this rank's block of C; all
        contiguous host tensors (pinned, for the copies to be asynchronous)."""
        torch, dist = self._torch, self._dist
        cs = stream if stream is not None else torch.cuda.current_stream()
        r0, r1 = self.share
        with torch.cuda.stream(cs):
            self.dA.copy_(hA, non_blocking=True)
            mine = self.dB[r0:r1]
            mine.copy_(hB[r0:r1], non_blocking=True)
            if self.world_size > 1:
                dist.all_gather_into_tensor(self.dB, mine, group=self.group)   # in place
            self.plan.run(self.dA, self.dB, self.dC, cs)
            hC.copy_(self.dC, non_blocking=True)

    def destroy(self) -> None:
        if self.plan is not None:
            self.plan.destroy()
            self.plan = None


def split_bands(row0: int, row1: int, bands: int, align: int = 256,
                taper: bool = False) -> List[Tuple[int, int]]:
    """Cut the rows [row0, row1) of one rank's block into at most `bands` non-empty bands whose
    inner boundaries fall on multiples of `align` rows counted from row0 (one pair tile), the
    earlier bands taking the remainder units. With `taper` the bands shrink towards the end
    (sizes in proportion bands : bands-1 : ... : 1): only the last band's copy is exposed, so it
    should be the smallest, while the early bands stay large enough to fill the device."""
    if bands < 1:
        raise ValueError("bands must be positive")
    if not taper:
        return [(row0 + a, row0 + b) for a, b in _split(row1 - row0, bands, align) if b > a]
    extent = row1 - row0
    units = -(-extent // align)
    weights = list(range(bands, 0, -1))
    sizes = [units * w // sum(weights) for w in weights]
    for i in range(units - sum(sizes)):          # leftover units go to the earliest bands
        sizes[i % bands] += 1
    if units >= bands:                           # every band gets at least one unit
        for i in range(bands - 1, 0, -1):
            if sizes[i] == 0:
                j = max(range(i), key=lambda t: sizes[t])
                sizes[j] -= 1
                sizes[i] = 1
    sizes.sort(reverse=True)
    out, start = [], 0
    for n in sizes:
        stop = min(start + n * align, extent)
        if stop > start:
            out.append((row0 + start, row0 + stop))
        start = stop
    return out


def default_bands(rows: int, cols: int) -> int:
    """Bands per block for the overlapped exchange. More bands hide more of the copy but leave
    each kernel fewer 256 x 256 tiles to spread over the device (74 CTA pairs). Measured on
    B200s: blocks of 512 tiles (2048 x 16384, 4096 x 8192) are best cut in 4, blocks of 64 to 256
    tiles (1024 x 4096, 4096 x 4096) in 2."""
    tiles = -(-rows // 256) * -(-cols // 256)
    if tiles >= 384:
        return 4
    if tiles >= 48:
        return 2
    return 1


def push_order(rank: int, world_size: int, dest: str, root: int = 0) -> List[int]:
    """Ranks this rank pushes its finished bands to. "root": only the root (nothing when this
    rank is the root); "all": every other rank, starting with the next one so that at any
    moment the ranks write to different destinations instead of all converging on rank 0."""
    if dest == "root":
        return [] if rank == root else [root]
    if dest == "all":
        return [(rank + d) % world_size for d in range(1, world_size)]
    raise ValueError(f"dest must be 'root' or 'all', not {dest!r}")


# Flag array of the fused exchange (one per rank, in symmetric memory).
FLAG_WORDS = 64
FLAG_GO = 32


@dataclass(frozen=True)
class BandStep:
    """One band of a rank's block in the overlapped exchange: the kernel computes rows
    [row0, row1) of C, then the band is copied to every rank in `dests`. Offsets are in
    elements: `a_off` into the rank's A rows, `b_off` into B (the block's first column), `c_off`
    into the full C (the band's first element; the same in every rank's copy of C)."""
    row0: int
    row1: int
    cols: int
    a_off: int
    b_off: int
    c_off: int
    dests: Tuple[int, ...]


def band_schedule(block: Block, N: int, K: int, bands: int, dests: Sequence[int],
                  taper: bool = False) -> List[BandStep]:
    """The steps of one rank: its block cut by `split_bands`, each band with its operand and
    output offsets and the ranks it is pushed to."""
    if block.cols <= 0:
        return []
    return [BandStep(r0, r1, block.cols, (r0 - block.row0) * K, block.col0, r0 * N + block.col0,
                     tuple(dests))
            for r0, r1 in split_bands(block.row0, block.row1, bands, taper=taper)]


# Steps a pipelined fused exchange can count (the arrival flags are copied from a table).
STEP_TABLE = 1 << 20

# What the TMA units of several GPUs together push into one GPU's memory over NVLink (measured
# on B200 / NVSwitch; a copy engine reaches 770).
PEER_STORE_GBS = 690.0


def fused_round_shape(ingress_bytes: int, kernel_ms: float, tiles: int, workers: int,
                      rounds: Optional[int] = None,
                      round_ratio: Optional[int] = None) -> Tuple[int, int]:
    """Rounds of the progressive schedule for a kernel whose C leaves over NVLink while it
    computes: (number of rounds, size of each round relative to the previous one in percent).

    With a = t_link / t_compute: for a < 1 (the computation is the longer of the two) little
    should be left to send when the kernel ends, so the rounds shrink; for a > 1 the link is the
    bottleneck and should start early, so they grow. On paper rounds in a geometric sequence of
    ratio a are ideal -- every round's output has just left when the next one's arrives -- but
    every round in which a tile is shared by several workers costs 10-25 us of exchange, while
    rounds of more tiles than workers are nearly free. Measured on 4 and 8 B200s (8192 x 4096 x
    4096 and 16384^3 sharded by rows; rounds 1-8, ratios 40-250 %), the best shapes were:
    a block of many waves (tiles >= 4 x workers): no rounds at all (0) -- whole tiles already
    leave wave after wave, and cutting them costs more than the shorter tail saves (16384^3 on
    2 GPUs in 16 rounds: 17.4 ms against 16.2 for the kernels alone; 7.1 against 5.8 in
    1xTF32); a block of one to four waves: two rounds, the second 40 % of the
    first, when the computation dominates, four rounds growing by 160 % when the link does; a
    block of less than one wave (every round shares its tiles): four equal rounds.
    `ingress_bytes` is what all senders together push into the collecting GPU, `kernel_ms` one
    sender's kernel time, `tiles` and `workers` the block's tile count and the CTAs (or CTA
    pairs) of the grid."""
    link_ms = ingress_bytes / (PEER_STORE_GBS * 1e6)
    a = link_ms / max(kernel_ms, 1e-6)
    if tiles >= 4 * workers:
        shape = (0, 100)
    elif tiles < workers:
        shape = (4, 100)
    else:
        shape = (2, 40) if a <= 1.0 else (4, 160)
    return (shape[0] if rounds is None else rounds,
            shape[1] if round_ratio is None else round_ratio)


class OverlappedGemm:
    """Sharded C = A @ B whose exchange of C runs underneath the computation.

    Every rank holds the whole C in symmetric memory (one allocation per rank, mapped into the
    other ranks' address spaces over NVLink). A rank computes its block band by band; as soon as
    a band is finished it is pushed into the destination ranks' C by the copy engines on side
    streams while the tensor cores work on the next band, so only the last band's copy is
    exposed. `finish` closes the step with one small all-reduce enqueued behind the copies: when
    it has completed on a rank, every rank's pushes had completed before it.

    dest = "root": the whole C ends up on `root` (a gather); dest = "all": on every rank.
    With `fused=True` (dest = "root" only) there are no bands, no copies and no collective:
    each rank runs one kernel over its whole block that writes its tiles straight into the
    root's C through the peer mapping. The kernel hands finished tiles to its TMA unit from a
    staging area in shared memory (so the warps that drain the accumulators never wait for
    NVLink) and follows the progressive schedule (`rounds`: all SMs work on a few tiles at a
    time, so finished tiles leave at a steady rate from the first microseconds on and the
    transfer runs underneath the rest of the computation instead of after it). The step is
    closed by flags: each rank stores a step counter into its word of the root's flag array
    once its stores have been performed, the root waits (bounded) for all of them, then releases
    the others into the next step by storing the counter into their "go" word, so that nobody
    overwrites a C that the root may still be reading. The kernel does both halves of a rank's
    hand-shake itself (`GemmPlan.run_synced_ptr`): it waits for "go" only in front of its first
    store, i.e. while the first tiles are being computed, and its last warp to finish raises
    the arrival flag, so no launch boundary lies between the last store and the flag. An rTile
    whose kernel lacks the staging area keeps the kernel's own stores and is bracketed by the
    two flag kernels instead.
    C must not be read while another rank may still be pushing the next step into it: on the
    root call `finish(release=False)`, enqueue the reader, then `release()` -- the "go" that lets
    the others overwrite the buffer. With `depth=2` (fused only) C alternates between two
    buffers and a sender waits for the "go" of the step before last, so the senders compute and
    push step s + 1 while the root still reads step s: consecutive jobs then take
    max(t_compute, t_link) each instead of their sum's exposed part (`og.C` is the buffer of
    the latest step).

        og = OverlappedGemm(M, N, K, rank, world, bands=4, dest="all")
        og.run(A_rows, B_full); og.finish()       # og.C now holds the product
    """

    def __init__(self, M: int, N: int, K: int, rank: int, world_size: int,
                 grid: Optional[Tuple[int, int]] = None, mode: int = 3,
                 bands: Optional[int] = None, dest: str = "root", root: int = 0, group=None, arch=None, measure: bool = False,
                 comm_streams: int = 2, taper: bool = False, fused: bool = False,
                 rounds: Optional[int] = None, round_ratio: Optional[int] = None,
                 wait_limit_cycles: int = 0, depth: int = 1):
        import os
        # plain peer mappings only: no NVLink multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib, roller
        from .analyze import MatmulConfig

        self.M, self.N, self.K = M, N, K
        self.rank, self.world_size = rank, world_size
        self.grid = grid if grid is not None else default_grid(world_size, M, N)
        if self.grid[0] * self.grid[1] != world_size:
            raise ValueError(f"grid {self.grid} does not match world size {world_size}")
        self.blocks = partition(M, N, self.grid[0], self.grid[1], align_m=256)
        self.block = self.blocks[rank]
        self.mode = mode
        self.group = group if group is not None else dist.group.WORLD
        if fused and dest != "root":
            raise ValueError("the fused output path delivers C to the root only")
        self.fused = fused
        self.root = root
        self.dests = push_order(rank, world_size, dest, root)
        self._lib = _lib
        self._dist = dist
        self._torch = torch

        if depth < 1 or (depth > 1 and not fused):
            raise ValueError("depth > 1 (several C buffers in flight) exists for the fused exchange only")
        # `depth` buffers for C, used in turn: with two, the senders already work on step s + 1
        # while the root still reads step s (they wait for "go" of step s + 1 - depth)
        self.depth = depth
        self.C_bufs = [symm_mem.empty((M, N), dtype=torch.float32, device=torch.device("cuda"))
                       for _ in range(depth)]
        self.handles = [symm_mem.rendezvous(c, self.group) for c in self.C_bufs]
        self.peer_C_bufs = [{d: h.get_buffer(d, (M, N), torch.float32) for d in self.dests}
                            for h in self.handles]
        self.handle = self.handles[0]
        self._token = torch.zeros(1, dtype=torch.float32, device="cuda")
        self._step = 0
        self._wait_limit = wait_limit_cycles
        if fused:
            if world_size > FLAG_GO:
                raise ValueError(f"the fused exchange handles at most {FLAG_GO} ranks")
            # words 0 .. world-1 of the root's array: "rank r's stores of step s have landed";
            # word FLAG_GO of every other rank's array: "the root is done with step s"
            self.flags = symm_mem.empty((FLAG_WORDS,), dtype=torch.int32, device=torch.device("cuda"))
            self.flags.zero_()
            torch.cuda.synchronize()
            self.flag_handle = symm_mem.rendezvous(self.flags, self.group)
            self.flag_status = torch.zeros(1, dtype=torch.int32, device="cuda")
            peers = range(world_size) if rank == root else (root,)
            self.peer_flags = {d: self.flag_handle.get_buffer(d, (FLAG_WORDS,), torch.int32)
                               for d in peers if d != rank}
            dist.barrier(group=self.group)     # every rank's flags are zero before anyone signals
        self.comm = [torch.cuda.Stream() for _ in range(max(1, comm_streams))]
        if fused:
            bands = 1
        if bands is None:
            bands = default_bands(self.block.rows, self.block.cols)
        self.steps = band_schedule(self.block, N, K, bands, self.dests, taper=taper)
        self.bands = [(st.row0, st.row1) for st in self.steps]
        self.plans, self.tiles, self._events = [], [], []
        self._synced = self._signalled = False
        self._pipe_plans, self._pipe_streams = None, None
        self.rounds = self.round_ratio = None
        by_shape = {}
        for r0, r1 in self.bands:
            shape = (r1 - r0, self.block.cols)
            if shape not in by_shape:
                cfg = MatmulConfig(shape[0], shape[1], K, _el_bits(mode))
                hint, fn, ms = roller.best_hint(cfg, arch, mode=mode, measure=measure)
                fn.plan.destroy()      # only the choice is kept; the bands get plans of their own
                by_shape[shape] = (roller.kernel_tile_for(hint), ms if ms else hint.est_us * 1e-3)
            tile, kernel_ms = by_shape[shape]
            self.tiles.append(tile)
            def new_plan(tile=tile, shape=shape, kernel_ms=kernel_ms):
                plan = _lib.GemmPlan(tile, shape[0], shape[1], K, lda=K, ldb=N, ldc=N, mode=mode)
                if fused and self.dests:
                    # C lives on the other side of NVLink: decoupled stores, steady tile completion
                    try:
                        plan.set_option(_lib.OPT_TMA_STORE, 1)
                        self._synced = True        # ... and the kernel does its own hand-shake
                        self.rounds, self.round_ratio = fused_round_shape(
                            self.block.rows * self.block.cols * 4 * (world_size - 1), kernel_ms,
                            -(-shape[0] // tile.block_m) * -(-shape[1] // tile.block_n),
                            _lib.device_info(torch.cuda.current_device()).sm_count // tile.cta_group,
                            rounds, round_ratio)
                        plan.set_option(_lib.OPT_PROGRESSIVE_ROUNDS, self.rounds)
                        plan.set_option(_lib.OPT_ROUND_RATIO, self.round_ratio)
                    except _lib.RollerError as e:
                        if e.status not in (_lib.ERR_UNSUPPORTED, _lib.ERR_INVALID):
                            raise
                if wait_limit_cycles:
                    plan.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, wait_limit_cycles)
                return plan

            self.plans.append(new_plan())
            self._events.append(torch.cuda.Event())
            if fused and depth > 1 and self.dests and self._synced:
                # Several steps in flight on a sending rank: a plan (scratch area, status word)
                # and a stream per C buffer. The kernels of consecutive steps share nothing but
                # the read-only operands, so they may run side by side: a CTA leaves as soon as
                # its last tile has been read from shared memory, the next step's CTA takes the
                # SM, and the arrival flag follows the kernel on its own stream once all its
                # stores have been performed. That flag is written by a copy engine (a 4-byte
                # copy of the step's number from a table on this GPU): a kernel could not run
                # before the next step's persistent CTAs, which fill every SM, have left.
                self._pipe_plans = [self.plans[0]] + [new_plan() for _ in range(depth - 1)]
                self.plans.extend(self._pipe_plans[1:])
                for p in self._pipe_plans:
                    p.set_option(_lib.OPT_EARLY_EXIT, 1)
                self._pipe_streams = [torch.cuda.Stream() for _ in range(depth)]
                self._step_table = torch.arange(1, STEP_TABLE + 1, dtype=torch.int32, device="cuda")

    def run(self, A_rows, B_full, stream=None) -> None:
        """Enqueue this rank's bands and their pushes. `A_rows` = A[rows of this rank's block, :]
        contiguous, `B_full` = the whole K x N matrix, contiguous."""
        torch = self._torch
        cs = stream if stream is not None else torch.cuda.current_stream()
        N = self.N
        eb = _el_bits(self.mode) // 8      # bytes per element of A and B; C is fp32
        for st in self.comm:
            st.wait_stream(cs)          # the previous step's consumers are ordered before the pushes
        n = 0
        if self.fused:
            self._step += 1
            # one kernel per rank; its C is the root's matrix (this rank's own on the root)
            peer_C = self.peer_C_bufs[(self._step - 1) % self.depth]
            out = peer_C[self.dests[0]] if self.dests else self.C
            step, plan = self.steps[0], self.plans[0]
            behind = self._step - self.depth       # the step whose C this one overwrites
            ptrs = (A_rows.data_ptr() + step.a_off * eb, B_full.data_ptr() + step.b_off * eb,
                    out.data_ptr() + step.c_off * 4)
            self._signalled = False
            if self._pipe_plans is not None:
                # (sending rank, several C buffers) this buffer's plan on this buffer's stream
                k = (self._step - 1) % self.depth
                st = self._pipe_streams[k]
                st.wait_stream(cs)            # the operands are ready
                self._pipe_plans[k].run_synced_ptr(
                    *ptrs, go_ptr=self.flags.data_ptr() + 4 * FLAG_GO if behind >= 1 else 0,
                    go_value=max(behind, 0), stream=st)
                if self._step > STEP_TABLE:
                    raise ValueError(f"the pipelined exchange counts at most {STEP_TABLE} steps")
                self._lib.copy_block_async(
                    self.peer_flags[self.root].data_ptr() + 4 * self.rank, 1,
                    self._step_table.data_ptr() + 4 * (self._step - 1), 1, 1, 1, st)
                self._signalled = True
                return
            if self.rank != self.root and self._synced:
                try:
                    # "go": the root has finished with the previous step's C; "arrive": this
                    # rank's stores of this step have landed
                    plan.run_synced_ptr(
                        *ptrs, go_ptr=self.flags.data_ptr() + 4 * FLAG_GO if behind >= 1 else 0,
                        go_value=max(behind, 0),
                        arrive_ptr=self.peer_flags[self.root].data_ptr() + 4 * self.rank,
                        arrive_value=self._step, stream=cs)
                    self._signalled = True
                    return
                except self._lib.RollerError as e:
                    if e.status != self._lib.ERR_UNSUPPORTED:
                        raise
                    self._synced = False
            if self.rank != self.root and behind >= 1:
                self._lib.flag_wait_async(self.flags.data_ptr(), FLAG_WORDS, 1 << FLAG_GO,
                                          behind, self.flag_status.data_ptr(),
                                          self._wait_limit, cs)
            plan.run_ptr(*ptrs, cs)
            return
        for step, plan, ev in zip(self.steps, self.plans, self._events):
            plan.run_ptr(A_rows.data_ptr() + step.a_off * eb, B_full.data_ptr() + step.b_off * eb,
                         self.C.data_ptr() + step.c_off * 4, cs)
            ev.record(cs)
            for d in step.dests:
                st = self.comm[n % len(self.comm)]
                n += 1
                st.wait_event(ev)
                self._lib.copy_block_async(self.peer_C[d].data_ptr() + step.c_off * 4, N,
                                           self.C.data_ptr() + step.c_off * 4, N,
                                           step.row1 - step.row0, step.cols, st)

    @property
    def C(self):
        """The matrix the current step delivers into (the last `run`'s; buffer 0 before any)."""
        return self.C_bufs[max(self._step - 1, 0) % self.depth]

    @property
    def peer_C(self):
        return self.peer_C_bufs[max(self._step - 1, 0) % self.depth]

    def release(self, stream=None) -> None:
        """Fused exchange, on the root: tell the other ranks that this step's C has been read
        (enqueued on `stream` behind the reader). `finish` does it right away unless called
        with `release=False`."""
        if not self.fused or self.rank != self.root:
            return
        cs = stream if stream is not None else self._torch.cuda.current_stream()
        others = [r for r in range(self.world_size) if r != self.root]
        if others:
            self._lib.flag_signal_async([self.peer_flags[r].data_ptr() + 4 * FLAG_GO
                                         for r in others], self._step, cs)

    def finish(self, stream=None, release: bool = True) -> None:
        """Enqueue the closing fence; once `stream` has passed it, every rank's pushes of this
        step have landed."""
        torch = self._torch
        cs = stream if stream is not None else torch.cuda.current_stream()
        if self.fused:
            if self.rank != self.root:
                if self._pipe_streams is not None:
                    # stay at most `depth` steps ahead of the caller's stream: it waits for the
                    # oldest step still in flight (the stream the next `run` will use)
                    cs.wait_stream(self._pipe_streams[self._step % self.depth])
                if self._signalled:
                    return      # the flag has been (or will be) raised behind the kernel
                # behind the kernel on the stream: its stores into the root's C have been performed
                self._lib.flag_signal_async([self.peer_flags[self.root].data_ptr() + 4 * self.rank],
                                            self._step, cs)
                return
            others = [r for r in range(self.world_size) if r != self.root]
            if others:
                mask = sum(1 << r for r in others)
                self._lib.flag_wait_async(self.flags.data_ptr(), FLAG_WORDS, mask, self._step,
                                          self.flag_status.data_ptr(), self._wait_limit, cs)
                if release:
                    self.release(cs)
            return
        lead = self.comm[0]
        for st in self.comm[1:]:
            lead.wait_stream(st)
        lead.wait_stream(cs)
        with torch.cuda.stream(lead):
            self._dist.all_reduce(self._token, group=self.group)
        cs.wait_stream(lead)

    def flops(self) -> int:
        return 2 * self.block.rows * self.block.cols * self.K

    def check_status(self) -> None:
        """Raises RollerError(TIMEOUT) when a kernel of this rank, or one of its waits for
        another rank's flag, gave up. Synchronises the device."""
        for p in self.plans:
            p.check_status()
        if self.fused:
            st = int(self.flag_status.item())
            if st != 0:
                self.flag_status.zero_()
                raise self._lib.RollerError(self._lib.ERR_TIMEOUT,
                                            f"wait for another rank's flag, status word = {st}")

    def destroy(self) -> None:
        for p in self.plans:
            p.destroy()
        self.plans = []
